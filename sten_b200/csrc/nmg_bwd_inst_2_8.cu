// Instances of the specialised SIMT transposed kernel for 2:8.
#include "nmg_spmm_t_simt_kernel.cuh"
namespace nmg {
template int simt_bwd_launch<2, 8>(int, const BwdParams &, const CUtensorMap &, int64_t, cudaStream_t);
}
