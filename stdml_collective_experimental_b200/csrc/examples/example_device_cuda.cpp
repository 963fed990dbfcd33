// The same session calls on CUDA device memory: pointers are told apart at run
// time, device buffers go through the fused sm_100a kernels over NVLink.
//   stdml_collective_run -np 2 example_device_cuda      (one GPU per rank)
// The reference's README lists a unified host/device interface as a TODO
// (README:9); this program is that interface at work.
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
    int ndev = 0;
    CUDA_OK(cudaGetDeviceCount(&ndev));
    const char *dev_env = std::getenv("STDML_COLLECTIVE_DEVICE_ID");
    CUDA_OK(cudaSetDevice((dev_env ? std::atoi(dev_env) : r) % ndev));

    const size_t count = 1 << 20;
    std::vector<float> host(count, float(r + 1));
    float *x = nullptr, *y = nullptr, *gathered = nullptr;
    CUDA_OK(cudaMalloc(&x, count * sizeof(float)));
    CUDA_OK(cudaMalloc(&y, count * sizeof(float)));
    CUDA_OK(cudaMalloc(&gathered, 4 * n * sizeof(float)));
    CUDA_OK(cudaMemcpy(x, host.data(), count * sizeof(float), cudaMemcpyHostToDevice));

    int bad = 0;
    sess.all_reduce(x, y, count, f32, sum, "grad");  // enqueued on the default stream
    CUDA_OK(cudaMemcpy(host.data(), y, count * sizeof(float), cudaMemcpyDeviceToHost));
    bad += host[0] != n * (n + 1) / 2.0f || host[count - 1] != n * (n + 1) / 2.0f;

    // a fused group with the 1/n scale applied in the kernel
    std::vector<workspace> ws;
    ws.push_back(workspace{x, x, 1000, f32, sum, "a"});
    ws.push_back(workspace{x + 1000, x + 1000, 77, f32, sum, "b"});
    ws.push_back(workspace{x + 2000, x + 2000, 500000, f32, sum, "c"});
    sess.group_all_reduce(ws, 1.0 / n);
    CUDA_OK(cudaMemcpy(host.data(), x, count * sizeof(float), cudaMemcpyDeviceToHost));
    bad += host[0] != (n + 1) / 2.0f || host[1076] != (n + 1) / 2.0f || host[2000 + 499999] != (n + 1) / 2.0f;
    bad += host[1077] != float(r + 1);  // outside the group: untouched

    sess.all_gather(y, gathered, 4, f32, "ag");
    std::vector<float> g(4 * n);
    CUDA_OK(cudaMemcpy(g.data(), gathered, g.size() * sizeof(float), cudaMemcpyDeviceToHost));
    for (float v : g) { bad += v != n * (n + 1) / 2.0f; }

    CUDA_OK(cudaMemset(y, 0, 16));
    sess.broadcast(x + 1077, y, 4, f32, "bc");  // rank 0's value everywhere
    CUDA_OK(cudaMemcpy(host.data(), y, 16, cudaMemcpyDeviceToHost));
    bad += host[0] != 1.0f;

    // gradients that live in the session's symmetric heap: tensors laid back to
    // back are reduced in place by ONE launch, nothing is packed or unpacked
    const size_t sizes[3] = {4096, 100000, 12};  // multiples of 4 floats: 16-byte boundaries
    float *heap = static_cast<float *>(sess.symm_alloc((4096 + 100000 + 12) * sizeof(float)));
    std::vector<float> ones(4096 + 100000 + 12, float(r + 1));
    CUDA_OK(cudaMemcpy(heap, ones.data(), ones.size() * sizeof(float), cudaMemcpyHostToDevice));
    std::vector<workspace> in_heap;
    size_t at = 0;
    for (const size_t s : sizes) {
        in_heap.push_back(workspace{heap + at, heap + at, s, f32, sum, "h" + std::to_string(at)});
        at += s;
    }
    const unsigned long long before = sess.device_launches();
    sess.group_all_reduce(in_heap, 1.0 / n);
    CUDA_OK(cudaMemcpy(ones.data(), heap, ones.size() * sizeof(float), cudaMemcpyDeviceToHost));
    bad += ones[0] != (n + 1) / 2.0f || ones.back() != (n + 1) / 2.0f;
    bad += sess.device_launches() - before != 1;
    sess.symm_free(heap);

    // separately allocated tensors, registered: their allocations are mapped on every
    // peer once, then ONE launch reduces them where they lie (no staging)
    if (n > 1) {
        sess.device_set_knob("register_min_bytes", 0);
        float *t[3] = {nullptr, nullptr, nullptr};
        const size_t len[3] = {1000, 77, 300001};
        std::vector<workspace> loose;
        for (int i = 0; i < 3; ++i) {
            CUDA_OK(cudaMalloc(&t[i], len[i] * sizeof(float)));
            std::vector<float> v(len[i], float(r + 1));
            CUDA_OK(cudaMemcpy(t[i], v.data(), len[i] * sizeof(float), cudaMemcpyHostToDevice));
            loose.push_back(workspace{t[i], t[i], len[i], f32, sum, "l" + std::to_string(i)});
        }
        const unsigned long long l0 = sess.device_launches();
        sess.group_all_reduce(loose, 1.0 / n);
        for (int i = 0; i < 3; ++i) {
            std::vector<float> v(len[i]);
            CUDA_OK(cudaMemcpy(v.data(), t[i], len[i] * sizeof(float), cudaMemcpyDeviceToHost));
            bad += v[0] != (n + 1) / 2.0f || v.back() != (n + 1) / 2.0f;
        }
        bad += sess.device_launches() - l0 != 1;
        sess.device_drop_registrations();  // before the tensors are freed
        sess.device_set_knob("register_min_bytes", -1);
        for (float *p : t) { cudaFree(p); }
    }

    std::printf("rank %d/%d on device memory: %s\n", r, n, bad == 0 ? "OK" : "WRONG");
    cudaFree(x);
    cudaFree(y);
    cudaFree(gathered);
    return bad == 0 ? 0 : 1;
}
