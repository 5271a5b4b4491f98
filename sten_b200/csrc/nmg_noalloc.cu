// nmg_spmm_noalloc: the SIMT forward matmul for callers that must not allocate device memory.
//
// Who needs it: code that runs where cudaMalloc is off limits -- inside a CUDA-graph capture or a stream-ordered
// region where an allocation would synchronise or invalidate the capture, in a process whose memory pool was
// sized up front and handed out completely (inference servers that pre-partition HBM), or in a latency-critical
// callback that may not take the allocator's locks.  Such a caller can still pass inputs and outputs it already
// owns, but it has nowhere to get the matmul's scratch (the fp32 [K][tokens] re-layout of the activation) from.
// Here the scratch lives in the library image itself: a file-scope device array of fixed size.
//
// Consequences the caller has to know:
//   * every GPU that loads the library holds NMG_NOALLOC_SCRATCH_BYTES of device memory until the process ends;
//   * problems whose scratch does not fit are rejected (NMG_ERR_UNSUPPORTED), they are never truncated;
//   * all calls on a device share the one array, and it keeps whatever the previous call left in it.  The kernels
//     overwrite every byte they later read, and the status word at its start is cleared at set-up, so stale
//     contents are harmless -- but two calls that overlap in time on the same GPU (different streams, different
//     threads) race on it and produce garbage.  Serialise them.
//   * the first call on a device resolves the array's device address (cudaGetSymbolAddress) and clears the status
//     word with a synchronous cudaMemset; make that first call before starting any stream capture.
//   * only (n, m) with a specialised kernel are served ({1:4, 2:4, 1:8, 2:8, 1:16, 3:6}); other patterns need a
//     device-side pattern table, which is an allocation.
// The entry point calls no cudaMalloc / cudaFree and no allocating library routine.
#include <mutex>

#include "nmg_spmm_simt.cuh"

namespace nmg {

// In host code this name is only a handle for the runtime (a host-side shadow symbol), not a device address: a
// kernel handed `g_noalloc_scratch` from the host would read the wrong memory.  The host obtains the real address
// with cudaGetSymbolAddress, once per device, below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[NMG_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
static std::mutex g_noalloc_mu;
static unsigned char *g_noalloc_ptr[kMaxDevices] = {};

// Device address of the array for the current device; first use per device does the set-up.
static int noalloc_scratch(unsigned char **out) {
    int dev = 0;
    NMG_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) NMG_FAIL(NMG_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    if (!g_noalloc_ptr[dev]) {
        void *p = nullptr;
        NMG_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
        if (!p) NMG_FAIL(NMG_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
        NMG_CUDA(cudaMemset(p, 0, 256));  // status word block must start at zero
        g_noalloc_ptr[dev] = static_cast<unsigned char *>(p);
    }
    *out = g_noalloc_ptr[dev];
    return NMG_OK;
}

int *noalloc_status_word(int dev) {
    if (dev < 0 || dev >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    return reinterpret_cast<int *>(g_noalloc_ptr[dev]);
}

}  // namespace nmg

using namespace nmg;

extern "C" int nmg_spmm_noalloc(const void *val, const int16_t *idx, int64_t M, int64_t K, int n, int m, int g,
                                int dtype, const void *act, int64_t ld_act, int64_t tokens, const void *bias,
                                void *out, int64_t ld_out, int layout, void *stream) {
    Geo geo;
    int rc = make_geo(M, K, n, m, g, &geo);
    if (rc) return rc;
    if (dtype != NMG_F32 && dtype != NMG_F16 && dtype != NMG_BF16) NMG_FAIL(NMG_ERR_INVALID, "unknown dtype %d", dtype);
    if (!val || !idx || !act || !out) NMG_FAIL(NMG_ERR_INVALID, "NULL operand pointer");
    if (n < 1 || tokens < 1) NMG_FAIL(NMG_ERR_INVALID, "n and tokens must be positive");
    if (layout != NMG_ACT_TOKEN_MAJOR && layout != NMG_ACT_K_MAJOR) NMG_FAIL(NMG_ERR_INVALID, "unknown activation layout %d", layout);
    const bool token_major = layout == NMG_ACT_TOKEN_MAJOR;
    if (ld_act < (token_major ? K : tokens)) NMG_FAIL(NMG_ERR_INVALID, "ld_act=%lld is smaller than the activation row", (long long)ld_act);
    if (ld_out < (token_major ? M : tokens)) NMG_FAIL(NMG_ERR_INVALID, "ld_out=%lld is smaller than the output row", (long long)ld_out);

    FwdChoice ch;
    int box_rows = 0, nbox = 0;
    if (!simt_fwd_specialised(n, m) || !choose_fwd(geo, dtype_size(dtype), &ch, &box_rows, &nbox))
        NMG_FAIL(NMG_ERR_UNSUPPORTED, "nmg_spmm_noalloc serves only n:m in {1:4, 2:4, 1:8, 2:8, 1:16, 3:6} with tiles that fit shared "
                                      "memory; %d:%d g=%d would need a device-side table allocation", n, m, g);
    const int64_t ld_xt = round_up(tokens, 128);
    const size_t need = 256 + (size_t)K * (size_t)ld_xt * 4;
    if (need > (size_t)NMG_NOALLOC_SCRATCH_BYTES)
        NMG_FAIL(NMG_ERR_UNSUPPORTED, "scratch of %zu bytes needed (256 + K * round_up(tokens,128) * 4) exceeds the built-in "
                                      "NMG_NOALLOC_SCRATCH_BYTES = %zu; use nmg_spmm with a caller-provided workspace",
                 need, (size_t)NMG_NOALLOC_SCRATCH_BYTES);

    unsigned char *scratch = nullptr;
    if ((rc = noalloc_scratch(&scratch))) return rc;
    int *status = reinterpret_cast<int *>(scratch);
    float *xt = reinterpret_cast<float *>(scratch + 256);
    cudaStream_t st = (cudaStream_t)stream;

    rc = token_major ? launch_transpose_to_f32(act, dtype, tokens, K, ld_act, xt, ld_xt, st)
                     : launch_widen_to_f32(act, dtype, K, tokens, ld_act, xt, ld_xt, st);
    if (rc) return rc;
    CUtensorMap tm;
    if ((rc = encode_tmap_2d(&tm, NMG_F32, xt, (uint64_t)ld_xt, (uint64_t)K, (uint64_t)ld_xt, (uint32_t)(32 * ch.tt), (uint32_t)box_rows, 0)))
        return rc;
    const int rbc = kWarps * (16 / m > 0 ? 16 / m : 1);
    FwdParams p{val, idx, bias, out, M, K, tokens, ld_out, geo.nb, geo.nc, g, geo.cc, box_rows, nbox, ch.stages, status};
    const size_t smem = fwd_smem_plan(geo.cc, n, rbc, 32 * ch.tt, nbox, box_rows, dtype_size(dtype), ch.stages).total;
    if (n == 1 && m == 4) return simt_fwd_launch<1, 4>(dtype, ch.tt, p, tm, rbc, smem, token_major, tokens, st);
    if (n == 2 && m == 4) return simt_fwd_launch<2, 4>(dtype, ch.tt, p, tm, rbc, smem, token_major, tokens, st);
    if (n == 1 && m == 8) return simt_fwd_launch<1, 8>(dtype, ch.tt, p, tm, rbc, smem, token_major, tokens, st);
    if (n == 2 && m == 8) return simt_fwd_launch<2, 8>(dtype, ch.tt, p, tm, rbc, smem, token_major, tokens, st);
    if (n == 1 && m == 16) return simt_fwd_launch<1, 16>(dtype, ch.tt, p, tm, rbc, smem, token_major, tokens, st);
    if (n == 3 && m == 6) return simt_fwd_launch<3, 6>(dtype, ch.tt, p, tm, rbc, smem, token_major, tokens, st);
    NMG_FAIL(NMG_ERR_UNSUPPORTED, "no specialised kernel for %d:%d", n, m);
}
