// send / recv of CUDA device buffers through the session: NCCL p2p on the
// session's own stream, beside an all_reduce on the default stream.
//   stdml_collective_run -np N test_send_recv_cuda     (N >= 2, one GPU per rank)
// Every rank sends a buffer to the next rank and receives from the previous one
// (even ranks send first, odd ranks receive first, so no two ranks wait for
// each other), with the async forms overlapping an all_reduce; then the same
// with the blocking forms, a 16-bit integer type (moved as bytes) and a host
// buffer (which still takes the TCP path).
#include <cstdio>
#include <vector>

#include <cuda_runtime.h>

#include <stdml/collective>

using namespace stdml::collective;

#define CUDA_OK(e)                                                             \
    do {                                                                       \
        const cudaError_t err_ = (e);                                          \
        if (err_ != cudaSuccess) {                                             \
            std::fprintf(stderr, "%s:%d %s\n", __FILE__, __LINE__, cudaGetErrorString(err_)); \
            return 2;                                                          \
        }                                                                      \
    } while (0)

int main()
{
    auto p = peer::from_env();
    session sess = p.join();
    const int n = static_cast<int>(sess.size()), r = static_cast<int>(sess.rank());
    if (n < 2) {
        std::printf("rank 0/1: needs two ranks\n");
        return 0;
    }
    int ndev = 0;
    CUDA_OK(cudaGetDeviceCount(&ndev));
    const char *dev_env = std::getenv("STDML_COLLECTIVE_DEVICE_ID");
    CUDA_OK(cudaSetDevice((dev_env ? std::atoi(dev_env) : r) % ndev));
    const size_t next = (r + 1) % n, prev = (r + n - 1) % n;
    const size_t count = 1 << 22;
    float *out = nullptr, *in = nullptr, *busy = nullptr;
    CUDA_OK(cudaMalloc(&out, count * 4));
    CUDA_OK(cudaMalloc(&in, count * 4));
    CUDA_OK(cudaMalloc(&busy, count * 4));
    std::vector<float> h(count, float(r + 1));
    CUDA_OK(cudaMemcpy(out, h.data(), count * 4, cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(busy, h.data(), count * 4, cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemset(in, 0, count * 4));
    int bad = 0;

    // async: transfers on the session's stream, an all_reduce on the default stream
    std::unique_ptr<task> ts, tr;
    if (r % 2 == 0) {
        ts = sess.async_send(out, count, f32, next, "ring");
        tr = sess.async_recv(in, count, f32, prev, "ring");
    } else {
        tr = sess.async_recv(in, count, f32, prev, "ring");
        ts = sess.async_send(out, count, f32, next, "ring");
    }
    sess.all_reduce(busy, busy, count, f32, sum, "busy");
    ts->finish();
    tr->finish();
    CUDA_OK(cudaDeviceSynchronize());
    CUDA_OK(cudaMemcpy(h.data(), in, count * 4, cudaMemcpyDeviceToHost));
    bad += h[0] != float(prev + 1) || h[count - 1] != float(prev + 1);
    CUDA_OK(cudaMemcpy(h.data(), busy, count * 4, cudaMemcpyDeviceToHost));
    bad += h[0] != float(n * (n + 1) / 2) || h[count / 2] != h[0];

    // blocking forms, int16 (NCCL has no such type: moved as bytes)
    int16_t *a16 = nullptr, *b16 = nullptr;
    CUDA_OK(cudaMalloc(&a16, 1001 * 2));
    CUDA_OK(cudaMalloc(&b16, 1001 * 2));
    std::vector<int16_t> h16(1001, int16_t(100 + r));
    CUDA_OK(cudaMemcpy(a16, h16.data(), 1001 * 2, cudaMemcpyHostToDevice));
    if (r % 2 == 0) {
        sess.send(a16, 1001, i16, next, "i16");
        sess.recv(b16, 1001, i16, prev, "i16");
    } else {
        sess.recv(b16, 1001, i16, prev, "i16");
        sess.send(a16, 1001, i16, next, "i16");
    }
    CUDA_OK(cudaMemcpy(h16.data(), b16, 1001 * 2, cudaMemcpyDeviceToHost));
    bad += h16[0] != int16_t(100 + prev) || h16[1000] != h16[0];

    // host buffers keep the TCP path
    int32_t hs = 7 * (r + 1), hr = 0;
    if (r % 2 == 0) {
        sess.send(&hs, 1, i32, next, "host");
        sess.recv(&hr, 1, i32, prev, "host");
    } else {
        sess.recv(&hr, 1, i32, prev, "host");
        sess.send(&hs, 1, i32, next, "host");
    }
    bad += hr != int32_t(7 * (prev + 1));

    std::printf("rank %d/%d send/recv of device buffers: %s\n", r, n, bad == 0 ? "OK" : "WRONG");
    cudaFree(out);
    cudaFree(in);
    cudaFree(busy);
    cudaFree(a16);
    cudaFree(b16);
    return bad == 0 ? 0 : 1;
}
