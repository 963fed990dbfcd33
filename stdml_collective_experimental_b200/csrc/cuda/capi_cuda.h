/* C ABI of the device (NVLink) data plane.  Pointer arguments named in/out/
 * ins/outs are arrays with one entry per virtual rank (one entry for a real
 * multi-GPU world); dtype and op values are those of
 * stdml/bits/collective/dtype.hpp.  The reference has no C interface to device
 * memory; its only C interface is the MPI facade (include/stdml/mpi.h). */
#ifndef STDML_COLLECTIVE_CAPI_CUDA_H
#define STDML_COLLECTIVE_CAPI_CUDA_H
#ifdef __cplusplus
extern "C" {
#endif

enum {
    STDMLC_OK = 0,
    STDMLC_ERR_RUNTIME = 1,
    STDMLC_ERR_ARGS = 2,
    STDMLC_ERR_NOMEM = 3,
    STDMLC_ERR_TIMEOUT = 4,
    STDMLC_ERR_PEER = 5, /* host path: a peer has gone (its connections closed) */
};

enum {
    STDMLC_INFO_RANK = 0,
    STDMLC_INFO_WORLD = 1,
    STDMLC_INFO_VRANKS = 2,
    STDMLC_INFO_HAS_NVLS = 3,
    STDMLC_INFO_ARENA_BYTES = 4,
    STDMLC_INFO_STAGING_BYTES = 5,
    STDMLC_INFO_LAUNCHES = 6,
    STDMLC_INFO_BACKEND = 7, /* 0 loopback, 1 vmm, 2 ipc */
};

const char *stdmlc_last_error(void);
int stdmlc_cuda_device_count(void);
int stdmlc_pointer_kind(const void *p);

int stdmlc_dw_create(void **out, int rank, int world, int device, int loopback,
                     unsigned long long heap_bytes, unsigned long long staging_bytes,
                     const char *key, const char *backend, int enable_nvls, int setup_timeout_ms,
                     unsigned long long wait_timeout_ms);
int stdmlc_dw_destroy(void *h);
int stdmlc_dw_info(void *h, int what, unsigned long long *out);
int stdmlc_dw_alloc(void *h, unsigned long long bytes, unsigned long long *off);
int stdmlc_dw_release(void *h, unsigned long long off);
int stdmlc_dw_ptr(void *h, int rank, unsigned long long off, void **out);
int stdmlc_dw_mc_ptr(void *h, unsigned long long off, void **out);
int stdmlc_dw_set_tuning(void *h, int max_blocks, long long oneshot_max_bytes,
                         long long nvls_oneshot_max_bytes, long long wait_timeout_ms);

/* Named knobs (same value on every rank): nvls_variant, nvls_blocks, tma_blocks,
 * tma_tile_vec, tma_min_bytes, tma_over_nvls_min_bytes, debug_checks. */
int stdmlc_dw_set_knob(void *h, const char *name, long long value);
/* Collective: unmap every peer buffer that registered calls have mapped
 * (register_min_bytes knob); call it before such memory is freed. */
int stdmlc_dw_drop_registrations(void *h);

int stdmlc_dw_all_reduce(void *h, const void *const *in, void *const *out,
                         unsigned long long count, int dt, int op, double scale, int algo,
                         void *stream);
int stdmlc_dw_reduce(void *h, const void *const *in, void *const *out, unsigned long long count,
                     int dt, int op, int root, double scale, void *stream);
int stdmlc_dw_group_all_reduce(void *h, unsigned long long n, const void *const *ins,
                               void *const *outs, const unsigned long long *counts, int dt, int op,
                               int user_dt, double scale, int algo, void *stream);
int stdmlc_dw_all_gather(void *h, const void *const *in, void *const *out,
                         unsigned long long count, int dt, void *stream);
int stdmlc_dw_broadcast(void *h, const void *const *in, void *const *out,
                        unsigned long long count, int dt, int root, void *stream);
int stdmlc_dw_barrier(void *h, void *stream);
/* Loopback worlds: barrier among the first `rows` virtual ranks only (rows <
 * world makes the bounded wait run out; see stdmlc_dw_status). */
int stdmlc_dw_barrier_rows(void *h, int rows, void *stream);
/* Launches the kernel as given (no staging, no chunking): for tests and tuning. */
int stdmlc_dw_raw_all_reduce(void *h, unsigned long long off, const void *const *src,
                             void *const *dst, unsigned long long count, int dt, int op, int algo,
                             int blocks, int root, int end_barrier, int has_scale, double scale,
                             void *stream);
int stdmlc_dw_status(void *h, int *out7);
int stdmlc_dw_check(void *h);
int stdmlc_dw_recover(void *h);

#ifdef __cplusplus
}
#endif
#endif
