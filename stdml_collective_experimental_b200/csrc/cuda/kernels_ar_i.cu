// All-reduce kernel instantiations for the signed integer wire types.
#include "ar_kernel.cuh"

namespace stdml::collective::cuda
{
int launch_all_reduce_i(const CommCtx &ctx, const AllReduceArgs &a, int dt, int op, int blocks,
                        int vranks, void *stream)
{
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dt) {
    case DT_I8:
        return launch_ops<DT_I8>(ctx, a, op, blocks, vranks, s);
    case DT_I16:
        return launch_ops<DT_I16>(ctx, a, op, blocks, vranks, s);
    case DT_I32:
        return launch_ops<DT_I32>(ctx, a, op, blocks, vranks, s);
    case DT_I64:
        return launch_ops<DT_I64>(ctx, a, op, blocks, vranks, s);
    }
    return -1;
}
}  // namespace stdml::collective::cuda
