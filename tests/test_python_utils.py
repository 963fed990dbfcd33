"""CPU tests of the pure-Python pieces: gradient-set shapes, trace parsing, NUMA
list parsing, the clock sampler against a fake NVML, custom-op registration."""
import os
import subprocess
import sys
import types

import torch

from stdml_collective_experimental_b200.models import gradsets
from stdml_collective_experimental_b200.models.resnet import ResNet50
from stdml_collective_experimental_b200.utils import clocks, numa, timeline

HERE = os.path.dirname(os.path.abspath(__file__))


def test_gradient_sets_match_the_named_models(tmp_path):
    r = gradsets.gradset_sizes("resnet50")
    assert (len(r), sum(r)) == (161, 25_557_032)
    v = gradsets.gradset_sizes("vgg16")
    assert (len(v), sum(v)) == (32, 138_357_544) and max(v) == 25088 * 4096
    b = gradsets.gradset_sizes("bert-base")
    assert len(b) == 199 and 109_000_000 < sum(b) < 110_000_000
    assert len(gradsets.gradset_sizes("bert-large")) == 391
    assert gradsets.gradset_sizes("1024x100") == [1024] * 100
    # the sets the reference's own files describe (testdata/resnet50.txt, bert.txt there)
    r214 = gradsets.gradset_sizes("resnet50-214")
    assert (len(r214), sum(r214)) == (214, 25_583_592)
    b599 = gradsets.gradset_sizes("bert-599")
    assert (len(b599), sum(b599)) == (599, 327_270_150)
    assert len(gradsets.SWEEP) == 9 and all("x" in w for w in gradsets.SWEEP)
    path = gradsets.write_sizes_file("resnet50", str(tmp_path / "r.txt"))
    assert [int(x) for x in open(path).read().split()] == r
    model = ResNet50()
    assert sorted(p.numel() for p in model.parameters()) == sorted(r)
    # the other benchmark models carry exactly their gradient sets too
    from stdml_collective_experimental_b200.models.bert import Bert, bert_base, bert_large
    from stdml_collective_experimental_b200.models.vgg import VGG16
    with torch.device("meta"):
        assert sorted(p.numel() for p in VGG16().parameters()) == sorted(v)
        assert sorted(p.numel() for p in bert_base().parameters()) == sorted(b)
        assert sorted(p.numel() for p in bert_large().parameters()) == \
            sorted(gradsets.gradset_sizes("bert-large"))
    # a small BERT runs, every parameter gets a gradient, padding does not leak
    torch.manual_seed(0)
    tiny = Bert(2, 64, 4, 128, vocab=100, max_pos=32, dropout=0.0)
    ids = torch.randint(0, 100, (3, 16))
    mask = torch.ones(3, 16)
    mask[:, 10:] = 0
    seq, pooled = tiny(ids, mask=mask)
    (seq.sum() + pooled.sum()).backward()
    assert seq.shape == (3, 16, 64) and pooled.shape == (3, 64)
    assert all(p.grad is not None for p in tiny.parameters())
    other = ids.clone()
    other[:, 10:] = 7
    assert torch.allclose(tiny(other, mask=mask)[0][:, :10], seq[:, :10], atol=1e-5)
    assert VGG16(num_classes=10)(torch.randn(1, 3, 32, 32)).shape == (1, 10)


def test_trace_lines_round_trip_through_the_native_runtime(tmp_path):
    from stdml_collective_experimental_b200 import _native
    _native.build()
    env = dict(os.environ, STDML_COLLECTIVE_ENABLE_TRACE="1")
    for k in ("KUNGFU_SELF_SPEC", "RANK", "WORLD_SIZE", "OMPI_COMM_WORLD_SIZE"):
        env.pop(k, None)
    out = subprocess.run([os.path.join(_native.CSRC, "build", "bin", "example_fork"), "2"], env=env,
                         stdout=subprocess.PIPE, text=True, timeout=120).stdout
    events = timeline.parse_log(out)
    names = {e["name"] for e in events}
    assert {"all_reduce", "send", "read_header"} <= names
    s = timeline.summary(events)
    assert s["all_reduce"]["calls"] >= 2 and s["send"]["bytes"] > 0
    trace = timeline.to_chrome_trace({0: events})
    assert trace["traceEvents"][0]["ph"] == "X"
    timeline.write_chrome_trace({0: events}, str(tmp_path / "t.json"))


def test_numa_cpulist_parsing():
    assert numa._parse_cpulist("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    assert numa._parse_cpulist("") == []
    assert numa.bind_to_gpu_numa(0) is None or isinstance(numa.bind_to_gpu_numa(0), int)


def test_clock_sampler_reads_but_never_sets(monkeypatch):
    calls = []

    fake = types.SimpleNamespace(
        NVML_CLOCK_SM=1,
        nvmlInit=lambda: calls.append("init"),
        nvmlDeviceGetHandleByIndex=lambda i: ("h", i),
        nvmlDeviceGetMaxClockInfo=lambda h, k: 1965,
        nvmlDeviceGetClockInfo=lambda h, k: 1350,
        nvmlDeviceGetCurrentClocksEventReasons=lambda h: 0x4,  # sw_power_cap
    )
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    s = clocks.ClockSampler(0, period_s=0.001).start()
    import time
    time.sleep(0.02)
    out = s.stop()
    assert out["sm_mhz"] == 1350 and out["sm_max_mhz"] == 1965 and out["reasons"] == ["sw_power_cap"]
    assert out["samples"] >= 2 and calls == ["init"]
    assert not [n for n in dir(fake) if "Set" in n or "Reset" in n]


def test_custom_ops_are_registered():
    from stdml_collective_experimental_b200.ops import torch_ops  # noqa: F401
    assert hasattr(torch.ops.stdml_collective, "all_reduce_")
    assert hasattr(torch.ops.stdml_collective, "group_all_reduce_")
    assert hasattr(torch.ops.stdml_collective, "all_gather")


def test_launcher_module_runs_a_job():
    out = subprocess.run([sys.executable, "-m", "stdml_collective_experimental_b200.run", "-q",
                          "-np", "2", "-runner-port", "38383", "-port-range", "10700",
                          sys.executable, "-c",
                          "from stdml_collective_experimental_b200.parallel import Peer\n"
                          "import torch\n"
                          "p = Peer.from_env(); s = p.join()\n"
                          "import os\n"
                          "v = int(s.all_reduce(torch.tensor([s.rank + 1]))[0])\n"
                          "os.write(1, ('sum %d\\n' % v).encode())\n"  # one write: ranks share the pipe
                          "s.close(); p.close()"],
                         stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300,
                         cwd=os.path.dirname(HERE))
    assert out.returncode == 0 and "sum 3" in out.stdout, out.stdout[-2000:]


def test_device_api_fails_loudly_without_a_gpu():
    import pytest
    if torch.cuda.is_available():
        pytest.skip("this checks the CPU-only behaviour")
    from stdml_collective_experimental_b200 import DeviceSession
    with pytest.raises(RuntimeError, match="no CUDA device"):
        DeviceSession.loopback(2)
    # the C++ session refuses device work the same way, host work is unaffected
    from stdml_collective_experimental_b200.parallel import Peer
    p = Peer.from_list(0, ["127.0.0.1:10880"])
    s = p.join()
    assert int(s.all_reduce(torch.tensor([5]))[0]) == 5
    s.close()
    p.close()


def test_native_api_reports_misuse_as_exceptions():
    import pytest
    from stdml_collective_experimental_b200 import _native
    from stdml_collective_experimental_b200.parallel import Peer, resized_cluster
    with pytest.raises(ValueError, match="malformed peer list"):
        Peer.from_list(0, ["not-an-address"])
    with pytest.raises(ValueError, match="rank outside"):
        Peer.from_list(3, ["127.0.0.1:10870"])
    with pytest.raises(ValueError):
        resized_cluster({"Runners": "oops"}, 2)
    grown = resized_cluster({"Runners": [{"IPv4": 2130706433, "Port": 38080}],
                             "Workers": [{"IPv4": 2130706433, "Port": 10000}]}, 3)
    assert [w["Port"] for w in grown["Workers"]] == [10000, 10001, 10002]
    p = Peer.from_list(0, ["127.0.0.1:10871"])
    s = p.join()
    with pytest.raises(ValueError, match="contiguous"):
        s.all_reduce(torch.ones(4, 4).t())
    with pytest.raises(ValueError, match="not defined"):
        s.all_reduce(torch.ones(4), op="bit_xor")
    with pytest.raises(ValueError, match="unknown reduce op"):
        s.all_reduce(torch.ones(4), op="avg")
    with pytest.raises(TypeError):
        s.all_reduce(torch.ones(4, dtype=torch.complex64))
    with pytest.raises(ValueError, match="must hold"):
        s.all_gather(torch.ones(4), torch.ones(5))
    assert _native.lib().stdmlc_dtype_size(8) == 2
    s.close()
    p.close()
    # null handles are errors with a message, never a crash; destroying null is a no-op
    import ctypes
    lib = _native.lib()
    v = ctypes.c_ulonglong()
    assert lib.stdmlc_session_info(None, 0, ctypes.byref(v)) == 2
    assert b"session handle" in lib.stdmlc_last_error()
    assert lib.stdmlc_session_barrier(None) == 2
    buf = ctypes.create_string_buffer(64)
    assert lib.stdmlc_peer_self(None, buf, 64) == 2 and b"peer handle" in lib.stdmlc_last_error()
    assert lib.stdmlc_dw_info(None, 0, ctypes.byref(v)) == 2
    assert lib.stdmlc_dw_destroy(None) == 0 and lib.stdmlc_peer_destroy(None) == 0


class _FakeStream:
    def __init__(self, *a, **k):
        pass

    def wait_event(self, ev):
        pass

    def wait_stream(self, s):
        pass

    def synchronize(self):
        pass


class _FakeEvent:
    def record(self, stream=None):
        pass


class _FakeSession:
    """Stands in for a 2-rank device session whose peer holds the same gradients:
    all_reduce(x, scale) -> x * 2 * scale, recorded call by call."""
    vranks, world, device = 1, 2, torch.device("cpu")

    def __init__(self):
        self.calls = []

    def symm_empty(self, n, dtype):
        return torch.empty(n, dtype=dtype)

    def symm_free(self, t):
        pass

    def all_reduce(self, t, scale=None, algo=None, stream=None):
        self.calls.append((t.data_ptr(), t.numel()))
        t.mul_(2.0 * (scale if scale is not None else 1.0))

    def broadcast(self, t, root=0):
        pass


def test_data_parallel_buckets_and_gradient_accumulation_on_cpu(monkeypatch):
    """The bucket bookkeeping of DataParallel (readiness order, one launch per
    bucket per synchronised backward, unused parameters, no_sync) does not
    depend on the GPU: run it with stand-ins for the streams and the session."""
    from stdml_collective_experimental_b200.parallel import ddp as ddp_mod

    monkeypatch.setattr(torch.cuda, "Stream", _FakeStream)
    monkeypatch.setattr(torch.cuda, "Event", _FakeEvent)
    monkeypatch.setattr(torch.cuda, "current_stream", lambda *a, **k: _FakeStream())

    torch.manual_seed(3)
    net = torch.nn.Sequential(torch.nn.Linear(5, 7), torch.nn.Tanh(), torch.nn.Linear(7, 3),
                              torch.nn.Tanh(), torch.nn.Linear(3, 2))
    unused = torch.nn.Parameter(torch.ones(9))  # never takes part in forward
    net.register_parameter("unused", unused)
    ref = torch.nn.Sequential(torch.nn.Linear(5, 7), torch.nn.Tanh(), torch.nn.Linear(7, 3),
                              torch.nn.Tanh(), torch.nn.Linear(3, 2))
    ref.load_state_dict({k: v for k, v in net.state_dict().items() if k != "unused"})

    sess = _FakeSession()
    dp = ddp_mod.DataParallel(net, sess, buckets=3)
    assert dp.nbuckets == 3
    # buckets tile the flat buffer, every tensor starts on a 16-byte boundary
    assert dp.bounds[0][0] == 0 and dp.bounds[-1][1] == dp.flat.numel()
    assert all(a[1] == b[0] for a, b in zip(dp.bounds, dp.bounds[1:]))
    assert all(p.grad.data_ptr() % 16 == dp.flat.data_ptr() % 16 for p in dp.params)

    x1, x2 = torch.randn(4, 5), torch.randn(4, 5)
    dp.zero_grad()
    dp(x1).square().sum().backward()
    assert len(sess.calls) == 3  # one launch per bucket, the unused parameter's bucket included
    assert [c[1] for c in sess.calls] == [hi - lo for lo, hi in dp.bounds]
    ref(x1).square().sum().backward()
    for (n, p) in net.named_parameters():
        if n != "unused":
            assert torch.allclose(p.grad, dict(ref.named_parameters())[n].grad, atol=1e-6), n
    assert torch.count_nonzero(unused.grad) == 0

    # accumulation: nothing is launched inside no_sync, the sum is reduced once afterwards
    sess.calls.clear()
    dp.zero_grad()
    ref.zero_grad()
    with dp.no_sync():
        dp(x1).square().sum().backward()
    assert sess.calls == []
    dp(x2).square().sum().backward()
    assert len(sess.calls) == 3
    ref(x1).square().sum().backward()
    ref(x2).square().sum().backward()
    for (n, p) in net.named_parameters():
        if n != "unused":
            assert torch.allclose(p.grad, dict(ref.named_parameters())[n].grad, atol=1e-6), n
    dp.close()
    assert all(p.grad is None for p in dp.params)


def test_host_reducer_against_plain_pytorch_reductions():
    """reduce_many is the oracle of every device test, so it is itself checked
    against reductions that share no code with it: float64 / int64 PyTorch
    arithmetic.  Integers, min and max must agree exactly; float sums and
    products within one rounding of the output type per accumulation step."""
    from stdml_collective_experimental_b200.utils.oracle import reduce_many
    g = torch.Generator().manual_seed(0)
    eps = {torch.float32: 2.0 ** -23, torch.float64: 2.0 ** -52, torch.bfloat16: 2.0 ** -7,
           torch.float16: 2.0 ** -10}
    for world in (1, 2, 3, 8):
        for dtype in (torch.float32, torch.float64, torch.bfloat16, torch.float16, torch.int8,
                      torch.int16, torch.int32, torch.int64, torch.uint8):
            n = 1027
            if dtype.is_floating_point:
                xs = [(torch.rand(n, generator=g) + 0.5).to(dtype) for _ in range(world)]
            else:
                info = torch.iinfo(dtype)
                xs = [torch.randint(max(info.min, -50), min(info.max, 50) + 1, (n,),
                                    generator=g).to(dtype) for _ in range(world)]
            wide = torch.stack([x.double() if dtype.is_floating_point else x.long() for x in xs])
            for op in ("sum", "min", "max", "prod") + (() if dtype.is_floating_point else ("bit_xor",)):
                got = reduce_many(xs, op)
                assert got.dtype == dtype
                if op == "min":
                    assert torch.equal(got, wide.min(0).values.to(dtype)), (dtype, op, world)
                elif op == "max":
                    assert torch.equal(got, wide.max(0).values.to(dtype)), (dtype, op, world)
                elif op == "bit_xor":
                    want = wide[0]
                    for w in wide[1:]:
                        want = want ^ w
                    assert torch.equal(got, want.to(dtype)), (dtype, world)
                elif not dtype.is_floating_point:
                    want = wide.sum(0) if op == "sum" else wide.prod(0)
                    bits = torch.iinfo(dtype).bits  # integer results wrap around
                    if dtype == torch.uint8:
                        want = want % 256
                    elif bits < 64:  # (values this small never leave int64)
                        want = (want + (1 << (bits - 1))) % (1 << bits) - (1 << (bits - 1))
                    assert torch.equal(got.long(), want), (dtype, op, world)
                else:
                    want = wide.sum(0) if op == "sum" else wide.prod(0)
                    # 16-bit floats: accumulated in f32, rounded once; others: one rounding a step
                    steps = 1 if dtype in (torch.bfloat16, torch.float16) else world
                    tol = eps[dtype] * steps * 1.01
                    assert torch.allclose(got.double(), want, rtol=tol, atol=0), (dtype, op, world)
            if dtype.is_floating_point:
                got = reduce_many(xs, "sum", 1.0 / 3.0)
                want = wide.sum(0) / 3.0
                steps = 2 if dtype in (torch.bfloat16, torch.float16) else world + 1
                assert torch.allclose(got.double(), want, rtol=eps[dtype] * steps * 1.01, atol=0)


def test_elastic_benchmark_refuses_to_drop_members_with_nvls_on(monkeypatch):
    """A rank must not leave a GPU job while its arena is bound to a multicast
    object: schedules that shrink need STDML_COLLECTIVE_NVLS=0, and say so."""
    import pytest
    from stdml_collective_experimental_b200.benchmarks import elastic
    assert elastic.shrinks(8, {50: 4, 100: 6, 150: 8})
    assert elastic.shrinks(4, {10: 6, 20: 5})
    assert not elastic.shrinks(2, {3: 4, 9: 4})
    assert not elastic.shrinks(6, {10: 4}, from_step=11)  # a joiner that arrives after the shrink

    class FakeSess:
        size = 8

    class FakePeer:
        self_id = "127.0.0.1:1"

    monkeypatch.delenv("STDML_COLLECTIVE_NVLS", raising=False)
    with pytest.raises(SystemExit) as e:
        elastic.run(None, FakePeer(), FakeSess(), {50: 4}, True, None)
    assert "STDML_COLLECTIVE_NVLS=0" in str(e.value)
