// Instances of the specialised SIMT transposed kernel for 1:4.
#include "nmg_spmm_t_simt_kernel.cuh"
namespace nmg {
template int simt_bwd_launch<1, 4>(int, const BwdParams &, const CUtensorMap &, int64_t, cudaStream_t);
}
