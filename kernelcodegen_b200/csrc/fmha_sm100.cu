#include "common.cuh"
namespace kcg {
size_t fmha_workspace_impl(const kcg_fmha_desc*) { return 0; }
kcg_status_t fmha_launch_impl(const kcg_fmha_desc*, const void*, const void*, const void*, void*, void*, size_t, cudaStream_t) { return KCG_UNSUPPORTED; }
}
