// group_all_reduce(vector<future<workspace>>) on CUDA device memory: the futures
// resolve late and in a different order on every rank (as the reference's own
// benchmark does it, benchmarks/bench_group_all_reduce.cpp:25-42,73-85), the
// tensors are reduced by fused launches over buckets cut from the list alone, so
// every rank issues the same launches in the same order.
//   test_group_futures_cuda                       one rank (one GPU)
//   stdml_collective_run -np N test_group_futures_cuda   N ranks, one GPU each
// Checks values exactly (small integers in f32 / i32) and the launch count.
#include <chrono>
#include <cstdio>
#include <future>
#include <random>
#include <thread>
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

    // 40 f32 tensors of 1 .. 6 MB, then 5 i32 tensors, then 3 more f32: with 64 MB
    // buckets that is a handful of f32 launches, one i32 launch, one f32 launch
    std::vector<size_t> counts;
    std::vector<dtype> types;
    for (int i = 0; i < 40; ++i) { counts.push_back(250000 + 1250000 * (i % 5) + i); types.push_back(f32); }
    for (int i = 0; i < 5; ++i) { counts.push_back(1000 + i); types.push_back(i32); }
    for (int i = 0; i < 3; ++i) { counts.push_back(77 + i); types.push_back(f32); }
    const size_t m = counts.size();

    size_t expected_launches = 0, fill = 0;
    for (size_t i = 0; i < m; ++i) {
        if (i > 0 && types[i] != types[i - 1] && fill > 0) { ++expected_launches; fill = 0; }
        fill += counts[i] * 4;
        if (fill >= session::group_bucket_bytes) { ++expected_launches; fill = 0; }
    }
    if (fill > 0) { ++expected_launches; }

    std::vector<void *> bufs(m);
    for (size_t i = 0; i < m; ++i) {
        CUDA_OK(cudaMalloc(&bufs[i], counts[i] * 4));
        if (types[i] == f32) {
            std::vector<float> h(counts[i], float((r + 1) * (int(i) % 7 + 1)));
            CUDA_OK(cudaMemcpy(bufs[i], h.data(), counts[i] * 4, cudaMemcpyHostToDevice));
        } else {
            std::vector<int32_t> h(counts[i], (r + 1) * (int(i) + 1));
            CUDA_OK(cudaMemcpy(bufs[i], h.data(), counts[i] * 4, cudaMemcpyHostToDevice));
        }
    }
    // warm the device path up (its first call builds the arena) so that the
    // launch count below belongs to the group alone
    void *scratch = nullptr;
    CUDA_OK(cudaMalloc(&scratch, 4096));
    CUDA_OK(cudaMemset(scratch, 0, 4096));
    sess.all_reduce(scratch, scratch, 1024, f32, stdml::collective::max, "warm");
    CUDA_OK(cudaDeviceSynchronize());
    cudaFree(scratch);
    const unsigned long long before = sess.device_launches();

    std::vector<std::promise<workspace>> promises(m);
    std::vector<std::future<workspace>> futures;
    for (auto &pr : promises) { futures.push_back(pr.get_future()); }
    // every rank resolves in its own order, a millisecond apart
    std::vector<size_t> order(m);
    for (size_t i = 0; i < m; ++i) { order[i] = i; }
    std::mt19937 rng(1234 + r);
    std::shuffle(order.begin(), order.end(), rng);
    std::thread resolver([&] {
        for (const size_t i : order) {
            std::this_thread::sleep_for(std::chrono::milliseconds(1));
            promises[i].set_value(
                workspace{bufs[i], bufs[i], counts[i], types[i], sum, "g" + std::to_string(i)});
        }
    });
    sess.group_all_reduce(std::move(futures));
    resolver.join();
    CUDA_OK(cudaDeviceSynchronize());
    const unsigned long long launches = sess.device_launches() - before;

    int bad = 0;
    const int tri = n * (n + 1) / 2;
    for (size_t i = 0; i < m; ++i) {
        if (types[i] == f32) {
            std::vector<float> h(counts[i]);
            CUDA_OK(cudaMemcpy(h.data(), bufs[i], counts[i] * 4, cudaMemcpyDeviceToHost));
            const float want = float(tri * (int(i) % 7 + 1));
            for (const size_t k : {size_t(0), counts[i] / 2, counts[i] - 1}) { bad += h[k] != want; }
        } else {
            std::vector<int32_t> h(counts[i]);
            CUDA_OK(cudaMemcpy(h.data(), bufs[i], counts[i] * 4, cudaMemcpyDeviceToHost));
            bad += h[0] != tri * (int(i) + 1) || h[counts[i] - 1] != h[0];
        }
        cudaFree(bufs[i]);
    }
    // tensors above the slot size are split over slots: at least one launch per
    // bucket, and the same number on every rank
    const unsigned long long lo = launches, hi = launches;
    unsigned long long mn = 0, mx = 0;
    sess.all_reduce(&lo, &mn, 1, u64, stdml::collective::min, "launches-min");
    sess.all_reduce(&hi, &mx, 1, u64, stdml::collective::max, "launches-max");
    if (mn != mx || launches < expected_launches || launches > 2 * expected_launches + 2) {
        std::printf("rank %d: %llu launches (ranks: %llu..%llu), %zu buckets expected\n", r, launches,
                    mn, mx, expected_launches);
        ++bad;
    }
    std::printf("rank %d/%d group_all_reduce(futures) on device memory: %s (%llu launches, %zu buckets)\n",
                r, n, bad == 0 ? "OK" : "WRONG", launches, expected_launches);
    return bad == 0 ? 0 : 1;
}
