// Instances of the specialised SIMT transposed kernel for 3:6.
#include "nmg_spmm_t_simt_kernel.cuh"
namespace nmg {
template int simt_bwd_launch<3, 6>(int, const BwdParams &, const CUtensorMap &, int64_t, cudaStream_t);
}
