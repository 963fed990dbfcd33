"""``DeviceSession``: collectives on CUDA tensors over NVLink peer memory.

One process per GPU (``DeviceSession.from_env``) or, for tests on a single GPU,
all ranks emulated on one device (``DeviceSession.loopback``).  In a loopback
session every tensor argument is a list with one tensor per emulated rank.

Semantics follow the reference's ``session``
(include/stdml/bits/collective/session.hpp:25-178): ``all_reduce`` with
sum/min/max/prod/bit_xor, rank-major ``all_gather``, ``broadcast`` (root 0 by
default, as the reference fixes it), plus ``reduce`` and a fused
``group_all_reduce`` with optional gradient scale and f32<->bf16/f16 cast.
"""
import ctypes
import os

import torch

from .. import _native

ALGO_ONESHOT, ALGO_TWOSHOT, ALGO_NVLS, ALGO_NVLS_ONESHOT, ALGO_TWOSHOT_TMA = 0, 1, 2, 3, 4
_ALGOS = {None: -1, "auto": -1, "oneshot": 0, "twoshot": 1, "nvls": 2, "nvls_oneshot": 3,
          "twoshot_tma": 4, "nvls_hybrid": 5}

_DTYPES = {
    torch.int8: 0, torch.int16: 1, torch.int32: 2, torch.int64: 3, torch.uint8: 4,
    torch.bfloat16: 8, torch.float16: 9, torch.float32: 10, torch.float64: 11,
}
for _name, _code in (("uint16", 5), ("uint32", 6), ("uint64", 7)):
    if hasattr(torch, _name):
        _DTYPES[getattr(torch, _name)] = _code
_OPS = {"sum": 0, "min": 1, "max": 2, "prod": 3, "bit_xor": 4, "xor": 4}


def dtype_code(dt):
    try:
        return _DTYPES[dt]
    except KeyError:
        raise TypeError(f"unsupported dtype {dt}") from None


def op_code(op):
    if isinstance(op, int):
        return op
    try:
        return _OPS[op]
    except KeyError:
        raise ValueError(f"unknown reduce op {op!r}") from None


def _algo_code(algo):
    if isinstance(algo, int):
        return algo
    try:
        return _ALGOS[algo]
    except KeyError:
        raise ValueError(f"unknown algorithm {algo!r}") from None


class _RawCuda:
    """Exposes a raw device range through the CUDA array interface."""

    def __init__(self, ptr, nbytes, owner):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}
        self._owner = owner


def _ptr_array(tensors):
    arr = (ctypes.c_void_p * len(tensors))()
    for i, t in enumerate(tensors):
        arr[i] = None if t is None else t.data_ptr()
    return arr


class DeviceSession:
    def __init__(self, handle, device):
        self._h = handle
        self._lib = _native.lib()
        self.device = torch.device("cuda", device)
        self.rank = self._info(0)
        self.world = self._info(1)
        self.vranks = self._info(2)
        self.loopback = self.vranks > 1 or (self.vranks == 1 and self._info(7) == 0)
        self._symm = []

    # ------------------------------------------------------------ construction
    @classmethod
    def _create(cls, rank, world, device, loopback, heap_bytes, staging_bytes, key, backend,
                enable_nvls, setup_timeout_ms, wait_timeout_ms):
        lib = _native.lib()
        if lib.stdmlc_cuda_device_count() <= 0:
            raise RuntimeError("no CUDA device: the device collectives need a B200")
        h = ctypes.c_void_p()
        torch.cuda.set_device(device)
        torch.cuda.init()
        _native.check(lib.stdmlc_dw_create(
            ctypes.byref(h), rank, world, device, 1 if loopback else 0, heap_bytes, staging_bytes,
            key.encode(), backend.encode(), 1 if enable_nvls else 0, setup_timeout_ms,
            wait_timeout_ms))
        return cls(h, device)

    @classmethod
    def loopback(cls, world, device=0, heap_bytes=64 << 20, staging_bytes=8 << 20,
                 wait_timeout_ms=5000):
        """All `world` ranks on one GPU (one cooperative launch per collective)."""
        return cls._create(0, world, device, True, heap_bytes, staging_bytes, "loopback", "auto",
                           False, 0, wait_timeout_ms)

    @classmethod
    def from_env(cls, heap_bytes=None, staging_bytes=None, key=None, backend=None,
                 enable_nvls=None, wait_timeout_ms=None, rank=None, world=None, device=None):
        """One rank of a multi-GPU world; RANK/WORLD_SIZE/LOCAL_RANK as set by torchrun."""
        env = os.environ
        rank = int(env.get("RANK", "0")) if rank is None else rank
        world = int(env.get("WORLD_SIZE", "1")) if world is None else world
        device = int(env.get("LOCAL_RANK", str(rank))) if device is None else device
        if heap_bytes is None:
            heap_bytes = int(env.get("STDML_COLLECTIVE_HEAP_MB", "1024")) << 20
        if staging_bytes is None:
            staging_bytes = int(env.get("STDML_COLLECTIVE_STAGING_MB", "64")) << 20
        if key is None:
            key = "%s.%s.%s" % (env.get("MASTER_PORT", "0"), env.get("TORCHELASTIC_RUN_ID", "x"),
                                env.get("STDML_COLLECTIVE_SESSION_KEY", "0"))
        if backend is None:
            backend = env.get("STDML_COLLECTIVE_SYMM", "auto")
        if enable_nvls is None:
            enable_nvls = env.get("STDML_COLLECTIVE_NVLS", "1") not in ("0", "false", "off")
        if wait_timeout_ms is None:
            wait_timeout_ms = int(env.get("STDML_COLLECTIVE_TIMEOUT_MS", "20000"))
        return cls._create(rank, world, device, False, heap_bytes, staging_bytes, key, backend,
                           enable_nvls, 120000, wait_timeout_ms)

    def close(self):
        if self._h is not None:
            self._symm.clear()
            h, self._h = self._h, None
            _native.check(self._lib.stdmlc_dw_destroy(h))

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---------------------------------------------------------------- queries
    def _info(self, what):
        v = ctypes.c_ulonglong()
        _native.check(self._lib.stdmlc_dw_info(self._h, what, ctypes.byref(v)))
        return int(v.value)

    @property
    def has_nvls(self):
        return bool(self._info(3))

    @property
    def backend(self):
        return {0: "loopback", 1: "vmm", 2: "ipc"}[self._info(7)]

    @property
    def staging_bytes(self):
        return self._info(5)

    @property
    def launches(self):
        """Kernels launched by this session so far."""
        return self._info(6)

    def set_tuning(self, max_blocks=0, oneshot_max_bytes=-1, nvls_oneshot_max_bytes=-1,
                   wait_timeout_ms=-1):
        _native.check(self._lib.stdmlc_dw_set_tuning(self._h, max_blocks, oneshot_max_bytes,
                                                     nvls_oneshot_max_bytes, wait_timeout_ms))

    def set_knob(self, name, value):
        """Named tuning knob, same value on every rank: nvls_variant (0..3),
        nvls_blocks, tma_blocks, tma_tile_vec, tma_min_bytes,
        tma_over_nvls_min_bytes (negative: never), gather_push_min_bytes, gather_mc,
        pipeline_min_bytes, debug_checks, group_bulk_min_bytes (registered groups of
        at least that many bytes load their operands with bulk asynchronous copies;
        negative: never), register_verify (0: a registered group trusts its tensors'
        addresses instead of looking up their allocation ids on every call), and register_min_bytes: collectives on
        ordinary CUDA tensors of at least that many bytes map the tensors'
        allocations on every peer (CUDA IPC, cached per allocation) and run
        zero-copy on them; negative: never (the default).  Tensors used that way
        must stay allocated until drop_registrations() or close()."""
        _native.check(self._lib.stdmlc_dw_set_knob(self._h, name.encode(), int(value)))

    def drop_registrations(self):
        """Collective: unmap every peer allocation that registered calls mapped.
        Call it before such memory goes back to the driver (for torch tensors:
        before torch.cuda.empty_cache())."""
        _native.check(self._lib.stdmlc_dw_drop_registrations(self._h))

    # ---------------------------------------------------------- symmetric heap
    def symm_empty(self, shape, dtype=torch.float32):
        """A tensor in the symmetric heap (collective: same calls on every rank).

        Collectives on such tensors are zero-copy.  Loopback: a list, one per rank."""
        if isinstance(shape, int):
            shape = (shape,)
        numel = 1
        for s in shape:
            numel *= int(s)
        nbytes = max(16, numel * torch.empty((), dtype=dtype).element_size())
        off = ctypes.c_ulonglong()
        _native.check(self._lib.stdmlc_dw_alloc(self._h, nbytes, ctypes.byref(off)))
        outs = []
        ranks = range(self.world) if self.vranks > 1 else [self.rank]
        for r in ranks:
            p = ctypes.c_void_p()
            _native.check(self._lib.stdmlc_dw_ptr(self._h, r, off.value, ctypes.byref(p)))
            raw = torch.as_tensor(_RawCuda(p.value, nbytes, self), device=self.device)
            t = raw.view(dtype)[:numel].view(*shape)
            t._stdml_arena_offset = off.value
            outs.append(t)
        self._symm.append(off.value)
        return outs if self.vranks > 1 else outs[0]

    def symm_free(self, tensor):
        t = tensor[0] if isinstance(tensor, (list, tuple)) else tensor
        off = t._stdml_arena_offset
        self._symm.remove(off)
        _native.check(self._lib.stdmlc_dw_release(self._h, off))

    # ------------------------------------------------------------- collectives
    def _per_rank(self, x, what):
        if self.vranks > 1:
            if not isinstance(x, (list, tuple)) or len(x) != self.vranks:
                raise ValueError(f"loopback session: {what} must be a list of {self.vranks} tensors")
            return list(x)
        return [x]

    @staticmethod
    def _checked(ts, what):
        for t in ts:
            if t is None:
                continue
            if not t.is_cuda:
                raise ValueError(f"{what}: CUDA tensor expected")
            if not t.is_contiguous():
                raise ValueError(f"{what}: contiguous tensor expected")
        return ts

    def _stream(self, stream):
        s = torch.cuda.current_stream(self.device) if stream is None else stream
        return ctypes.c_void_p(s.cuda_stream)

    def all_reduce(self, tensor, out=None, op="sum", scale=None, algo=None, stream=None):
        """out = scale * reduce(tensor over ranks); in place when `out` is None."""
        ins = self._checked(self._per_rank(tensor, "tensor"), "all_reduce")
        outs = ins if out is None else self._checked(self._per_rank(out, "out"), "all_reduce")
        t0 = ins[0]
        self._profiled("all_reduce", t0.numel() * t0.element_size(), stream,
                       lambda: _native.check(self._lib.stdmlc_dw_all_reduce(
                           self._h, _ptr_array(ins), _ptr_array(outs), t0.numel(),
                           dtype_code(t0.dtype), op_code(op),
                           1.0 if scale is None else float(scale), _algo_code(algo),
                           self._stream(stream))))
        return out if out is not None else tensor

    def reduce(self, tensor, out=None, op="sum", root=0, scale=None, stream=None):
        """Reduce to `root`; other ranks' `out` is left untouched (may be None)."""
        ins = self._checked(self._per_rank(tensor, "tensor"), "reduce")
        if out is None:
            outs = [t if (self.vranks > 1 and i == root) or (self.vranks == 1 and self.rank == root)
                    else None for i, t in enumerate(ins)]
        else:
            outs = self._checked(self._per_rank(out, "out"), "reduce")
        t0 = ins[0]
        _native.check(self._lib.stdmlc_dw_reduce(
            self._h, _ptr_array(ins), _ptr_array(outs), t0.numel(), dtype_code(t0.dtype),
            op_code(op), root, 1.0 if scale is None else float(scale), self._stream(stream)))
        return out if out is not None else tensor

    def group_all_reduce(self, tensors, outs=None, op="sum", scale=None, wire_dtype=None,
                         algo=None, stream=None):
        """Fused all-reduce of a whole list of tensors in one launch per staging slot.

        `wire_dtype` (bf16/f16) sends f32 tensors as 16-bit floats (cast fused into
        the pack/unpack phases).  Loopback: `tensors[rank][i]`."""
        # The same tensors are usually passed every step (a model's gradients):
        # the prepared pointer table is kept, keyed by every data pointer and
        # element count of the call, so a step costs one pass over the list and
        # one native call instead of the checks and conversions below.
        cache = getattr(self, "_group_cache", None)
        if cache is None:
            cache = self._group_cache = {}
        if outs is None and self.vranks == 1 and isinstance(tensors, list) and tensors:
            key = (tuple([t.data_ptr() for t in tensors]), tuple([t.numel() for t in tensors]),
                   tensors[0].dtype, wire_dtype)
            hit = cache.get(key)
            if hit is not None:
                n, arr, counts, wire, user, nbytes = hit
                self._profiled("group_all_reduce", nbytes, stream,
                               lambda: _native.check(self._lib.stdmlc_dw_group_all_reduce(
                                   self._h, n, arr, arr, counts, wire, op_code(op), user,
                                   1.0 if scale is None else float(scale), _algo_code(algo),
                                   self._stream(stream))))
                return tensors
        else:
            key = None
        per_rank = self._per_rank(tensors, "tensors") if self.vranks > 1 else [list(tensors)]
        per_rank_out = per_rank if outs is None else (
            self._per_rank(outs, "outs") if self.vranks > 1 else [list(outs)])
        n = len(per_rank[0])
        if n == 0:
            return outs if outs is not None else tensors
        dtypes = []
        for t in per_rank[0]:
            if t.dtype not in dtypes:
                dtypes.append(t.dtype)
        if len(dtypes) > 1:
            # one fused call per dtype, each keeping the callers' order
            for dt_ in dtypes:
                idx = [i for i, t in enumerate(per_rank[0]) if t.dtype == dt_]
                sub_in = [[pr[i] for i in idx] for pr in per_rank]
                sub_out = [[pr[i] for i in idx] for pr in per_rank_out]
                self.group_all_reduce(sub_in if self.vranks > 1 else sub_in[0],
                                      outs=None if outs is None else
                                      (sub_out if self.vranks > 1 else sub_out[0]),
                                      op=op, scale=scale,
                                      wire_dtype=wire_dtype if dt_ == torch.float32 else None,
                                      algo=algo, stream=stream)
            return outs if outs is not None else tensors
        dt = per_rank[0][0].dtype
        flat_in, flat_out = [], []
        for r in range(len(per_rank)):
            if len(per_rank[r]) != n or len(per_rank_out[r]) != n:
                raise ValueError("group_all_reduce: every rank needs the same number of tensors")
            for t in per_rank[r]:
                if t.dtype != dt:
                    raise ValueError("group_all_reduce: one dtype per call")
            flat_in += self._checked(list(per_rank[r]), "group_all_reduce")
            flat_out += self._checked(list(per_rank_out[r]), "group_all_reduce")
        counts = (ctypes.c_ulonglong * n)(*[t.numel() for t in per_rank[0]])
        if wire_dtype is None or wire_dtype == dt:
            wire, user = dtype_code(dt), -1
        else:
            wire, user = dtype_code(wire_dtype), dtype_code(dt)
        nbytes = sum(t.numel() * t.element_size() for t in per_rank[0])
        if key is not None:
            if len(cache) > 64:
                cache.clear()
            arr = _ptr_array(flat_in)
            cache[key] = (n, arr, counts, wire, user, nbytes)
        self._profiled("group_all_reduce", nbytes, stream,
                       lambda: _native.check(self._lib.stdmlc_dw_group_all_reduce(
                           self._h, n, _ptr_array(flat_in), _ptr_array(flat_out), counts, wire,
                           op_code(op), user, 1.0 if scale is None else float(scale),
                           _algo_code(algo), self._stream(stream))))
        return outs if outs is not None else tensors

    def all_gather(self, tensor, out, stream=None):
        """out[r * n:(r + 1) * n] = rank r's tensor (rank-major, as the reference)."""
        ins = self._checked(self._per_rank(tensor, "tensor"), "all_gather")
        outs = self._checked(self._per_rank(out, "out"), "all_gather")
        t0 = ins[0]
        if outs[0].numel() != t0.numel() * self.world:
            raise ValueError("all_gather: out must hold world * tensor.numel() elements")
        self._profiled("all_gather", t0.numel() * t0.element_size(), stream,
                       lambda: _native.check(self._lib.stdmlc_dw_all_gather(
                           self._h, _ptr_array(ins), _ptr_array(outs), t0.numel(),
                           dtype_code(t0.dtype), self._stream(stream))))
        return out

    def broadcast(self, tensor, out=None, root=0, stream=None):
        ins = self._checked(self._per_rank(tensor, "tensor"), "broadcast")
        outs = ins if out is None else self._checked(self._per_rank(out, "out"), "broadcast")
        t0 = ins[0]
        self._profiled("broadcast", t0.numel() * t0.element_size(), stream,
                       lambda: _native.check(self._lib.stdmlc_dw_broadcast(
                           self._h, _ptr_array(ins), _ptr_array(outs), t0.numel(),
                           dtype_code(t0.dtype), root, self._stream(stream))))
        return out if out is not None else tensor

    def barrier(self, stream=None):
        _native.check(self._lib.stdmlc_dw_barrier(self._h, self._stream(stream)))

    # ---------------------------------------------------------- point to point
    def _p2p_stream(self):
        if getattr(self, "_p2p", None) is None:
            self._p2p = torch.cuda.Stream(self.device)
        return self._p2p

    def send(self, tensor, dst):
        """Point-to-point send of a CUDA tensor: NCCL p2p (torch.distributed) on a
        stream of its own, so it overlaps the collectives of this session.  The
        reference's send/recv (src/stdml/collective/send_recv.cpp:6-21) is the
        rendezvous message of its TCP transport.  Returns a handle with wait()."""
        return self._p2p_op(tensor, dst, True)

    def recv(self, tensor, src):
        return self._p2p_op(tensor, src, False)

    def _p2p_op(self, tensor, peer, is_send):
        import torch.distributed as dist
        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("send/recv of CUDA tensors needs torch.distributed (backend nccl)")
        side = self._p2p_stream()
        cur = torch.cuda.current_stream(self.device)
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            if is_send:
                dist.send(tensor, peer)
            else:
                dist.recv(tensor, peer)
            done = torch.cuda.Event()
            done.record(side)
        tensor.record_stream(side)

        class _Handle:
            def wait(self_h, stream=None):
                (stream or torch.cuda.current_stream(self.device)).wait_event(done)

            def synchronize(self_h):
                done.synchronize()
        return _Handle()

    def barrier_rows(self, rows, stream=None):
        """Loopback only: barrier among the first `rows` emulated ranks.  With
        rows < world the others never arrive and the bounded wait runs out."""
        _native.check(self._lib.stdmlc_dw_barrier_rows(self._h, rows, self._stream(stream)))

    def raw_all_reduce(self, symm, src=None, dst=None, count=None, op="sum", algo=ALGO_TWOSHOT,
                       blocks=0, root=-1, end_barrier=False, scale=None, stream=None):
        """Launch the kernel exactly as given on a symmetric buffer (tests, tuning)."""
        sy = self._per_rank(symm, "symm")
        srcs = [None] * self.vranks if src is None else self._per_rank(src, "src")
        dsts = [None] * self.vranks if dst is None else self._per_rank(dst, "dst")
        n = sy[0].numel() if count is None else count
        _native.check(self._lib.stdmlc_dw_raw_all_reduce(
            self._h, sy[0]._stdml_arena_offset, _ptr_array(srcs), _ptr_array(dsts), n,
            dtype_code(sy[0].dtype), op_code(op), algo, blocks, root, 1 if end_barrier else 0,
            0 if scale is None else 1, 1.0 if scale is None else float(scale),
            self._stream(stream)))

    # --------------------------------------------------------------- profiling
    def enable_profile(self, on=True):
        """Record a CUDA event pair around every collective of this session (device
        time per call, no host synchronisation until profile_summary()).  The
        reference's counterpart is its STDML_COLLECTIVE_PROFILE_RATE scopes
        (include/stdml/bits/collective/stat.hpp:196-202), which time the host."""
        self._prof = [] if on else None

    def _profiled(self, name, nbytes, stream, call):
        prof = getattr(self, "_prof", None)
        if prof is None:
            return call()
        s = torch.cuda.current_stream(self.device) if stream is None else stream
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s)
        out = call()
        e1.record(s)
        prof.append((name, nbytes, e0, e1))
        return out

    def profile_summary(self, reset=True):
        """{op: {calls, bytes, ms, algbw_gb_s, busbw_gb_s}}; waits for the recorded work."""
        prof = getattr(self, "_prof", None) or []
        out = {}
        n = self.world
        factor = {"all_reduce": 2 * (n - 1) / n, "group_all_reduce": 2 * (n - 1) / n,
                  "all_gather": (n - 1), "broadcast": 1.0, "reduce": 1.0, "barrier": 0.0}
        for name, nbytes, e0, e1 in prof:
            e1.synchronize()
            d = out.setdefault(name, {"calls": 0, "bytes": 0, "ms": 0.0})
            d["calls"] += 1
            d["bytes"] += nbytes
            d["ms"] += e0.elapsed_time(e1)
        for name, d in out.items():
            sec = max(d["ms"], 1e-9) * 1e-3
            d["algbw_gb_s"] = d["bytes"] / sec / 1e9
            d["busbw_gb_s"] = d["algbw_gb_s"] * factor.get(name, 1.0)
        if reset and getattr(self, "_prof", None) is not None:
            self._prof = []
        return out

    # ------------------------------------------------------------ failure path
    def status(self):
        """(code, rank, block, peer, phase, want, have); code 0 = healthy.  Never blocks."""
        out = (ctypes.c_int * 7)()
        _native.check(self._lib.stdmlc_dw_status(self._h, out))
        return tuple(out)

    def check(self):
        """Raise DeviceTimeoutError if a kernel gave up waiting for a peer."""
        _native.check(self._lib.stdmlc_dw_check(self._h))

    def recover(self):
        """Collective: clear the signal pads after a timeout so the session is usable again."""
        _native.check(self._lib.stdmlc_dw_recover(self._h))
