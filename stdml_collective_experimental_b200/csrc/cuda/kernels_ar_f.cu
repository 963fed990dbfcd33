// All-reduce kernel instantiations for the floating-point wire types.
#include "ar_kernel.cuh"

namespace stdml::collective::cuda
{
int launch_all_reduce_f(const CommCtx &ctx, const AllReduceArgs &a, int dt, int op, int blocks,
                        int vranks, void *stream)
{
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dt) {
    case DT_BF16:
        return launch_ops<DT_BF16>(ctx, a, op, blocks, vranks, s);
    case DT_F16:
        return launch_ops<DT_F16>(ctx, a, op, blocks, vranks, s);
    case DT_F32:
        return launch_ops<DT_F32>(ctx, a, op, blocks, vranks, s);
    case DT_F64:
        return launch_ops<DT_F64>(ctx, a, op, blocks, vranks, s);
    }
    return -1;
}
}  // namespace stdml::collective::cuda
