/* stdmlc_all_reduce_noalloc: an all-reduce entry point that allocates nothing.
 *
 * This entry point has no counterpart in the reference (which has no device
 * code at all); it exists for callers of this library that are not allowed to
 * allocate device memory themselves or to trigger an allocation inside a
 * library call.  Typical cases: a plugin that runs inside a host application
 * whose device memory is owned entirely by that application's own allocator
 * (any cudaMalloc made behind its back breaks its memory accounting or is simply
 * forbidden by policy), and steady-state loops that must never hit the
 * implicit device-wide synchronisation that cudaMalloc / cudaFree perform.
 * The regular entry points (stdmlc_dw_create + stdmlc_dw_all_reduce) allocate a
 * symmetric arena, a status block and descriptor tables; this one does not.
 *
 * What it does: the single-GPU ("loopback") form of the fused all-reduce
 * kernel.  `nranks` input buffers that live on the current device, one per
 * emulated rank, are reduced element-wise in rank order and the result (times
 * `scale`, for floating-point types, when scale != 1) is written to each of the
 * `nranks` output buffers:  out[r][i] = scale * (in[0][i] op ... op in[n-1][i]).
 * in[r] == out[r] is allowed.  The kernel is the same one the loopback device
 * session launches; only its scratch memory differs.
 *
 * Scratch memory: the kernel needs a signal pad and a staging buffer per rank.
 * Here they live in ONE file-scope `static __device__` array of
 * STDMLC_NOALLOC_SCRATCH_BYTES bytes (5 MiB).  Every GPU on which this library
 * is loaded holds that array from the moment the module is loaded until the
 * process exits, whether or not this function is ever called.
 *
 * Limits (a call beyond them returns STDMLC_ERR_ARGS with a message in
 * stdmlc_last_error(), nothing is launched):
 *   1 <= nranks <= STDMLC_NOALLOC_MAX_RANKS (8);
 *   count * sizeof(element) <= STDMLC_NOALLOC_MAX_BYTES (512 KiB) per buffer;
 *   dt / op as in stdml/bits/collective/dtype.hpp (bit_xor: integers only).
 *
 * First call on a device: the address of the scratch array on that device is
 * looked up once (cudaGetSymbolAddress, with that device current) and kept.
 * This set-up happens inside the first call made while that device is current,
 * so make that first call before any stream capture begins on that device.
 *
 * Calls share the array.  Every call clears the signal pads itself (an
 * asynchronous memset on `stream`, ahead of the kernel); the staging area
 * keeps whatever the previous call left there and is overwritten before it is
 * read.  Two calls that overlap on the GPU (different streams, or the same
 * call from two threads) race on the array and give undefined results:
 * serialise them on one stream.
 *
 * The call is asynchronous: it returns after enqueuing a memset and one
 * cooperative kernel launch on `stream` (NULL = the legacy default stream).
 * It calls no cudaMalloc, cudaFree, cudaHostAlloc, nor any allocating library
 * routine.  Returns 0 on success.
 *
 * Learning of a failure: every wait inside the kernel is bounded (2 s).  A wait
 * that runs out (in practice: two calls overlapping on the GPU, against the
 * rule above) makes the kernel's blocks return early; the call itself returned
 * 0 long before.  The record of that is kept in device memory, because this
 * entry point may not allocate the pinned host memory that the regular
 * sessions use for it.  stdmlc_all_reduce_noalloc_status(out7, stream) copies
 * it back (one cudaMemcpyAsync on `stream` and a wait for that stream; no
 * allocation either): out7 = {code, rank, block, peer, phase, want, have},
 * code 0 = the calls enqueued on `stream` so far all completed.  It returns 0
 * when healthy and STDMLC_ERR_TIMEOUT (4) after a wait that ran out; the next
 * stdmlc_all_reduce_noalloc call clears the record. */
#ifndef STDML_COLLECTIVE_NOALLOC_ALL_REDUCE_H
#define STDML_COLLECTIVE_NOALLOC_ALL_REDUCE_H
#ifdef __cplusplus
extern "C" {
#endif

#define STDMLC_NOALLOC_MAX_RANKS 8
#define STDMLC_NOALLOC_MAX_BYTES (512u << 10)
#define STDMLC_NOALLOC_SCRATCH_BYTES (STDMLC_NOALLOC_MAX_RANKS * ((128u << 10) + STDMLC_NOALLOC_MAX_BYTES))

int stdmlc_all_reduce_noalloc(const void *const *in, void *const *out, int nranks,
                              unsigned long long count, int dt, int op, double scale,
                              void *stream);

int stdmlc_all_reduce_noalloc_status(int *out7, void *stream);

#ifdef __cplusplus
}
#endif
#endif
