// All-reduce kernel instantiations for the unsigned integer wire types.
#include "ar_kernel.cuh"

namespace stdml::collective::cuda
{
int launch_all_reduce_u(const CommCtx &ctx, const AllReduceArgs &a, int dt, int op, int blocks,
                        int vranks, void *stream)
{
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dt) {
    case DT_U8:
        return launch_ops<DT_U8>(ctx, a, op, blocks, vranks, s);
    case DT_U16:
        return launch_ops<DT_U16>(ctx, a, op, blocks, vranks, s);
    case DT_U32:
        return launch_ops<DT_U32>(ctx, a, op, blocks, vranks, s);
    case DT_U64:
        return launch_ops<DT_U64>(ctx, a, op, blocks, vranks, s);
    }
    return -1;
}
}  // namespace stdml::collective::cuda
