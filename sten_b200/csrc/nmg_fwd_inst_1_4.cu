// Instances of the specialised SIMT forward kernel for 1:4.
#include "nmg_spmm_simt_kernel.cuh"
namespace nmg {
template int simt_fwd_launch<1, 4>(int, int, const FwdParams &, const CUtensorMap &, int, size_t, bool, int64_t, cudaStream_t);
}
