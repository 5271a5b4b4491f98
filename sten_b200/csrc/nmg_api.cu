// C-ABI entry points of the matmul: argument validation and choice of kernel family.
#include "nmg_spmm_simt.cuh"

using namespace nmg;

static int check_common(int dtype, int64_t tokens, const void *a, const void *b, const void *c, const void *d) {
    if (dtype != NMG_F32 && dtype != NMG_F16 && dtype != NMG_BF16)
        NMG_FAIL(NMG_ERR_INVALID, "dtype must be NMG_F32, NMG_F16 or NMG_BF16, got %d", dtype);
    if (tokens < 1) NMG_FAIL(NMG_ERR_INVALID, "tokens must be positive, got %lld", (long long)tokens);
    if (!a || !b || !c || !d) NMG_FAIL(NMG_ERR_INVALID, "NULL operand pointer");
    return NMG_OK;
}

extern "C" size_t nmg_spmm_workspace_bytes(int64_t M, int64_t K, int64_t tokens, int n, int m, int g, int dtype,
                                           int layout, int algo) {
    Geo geo;
    if (make_geo(M, K, n, m, g, &geo) || tokens < 1) return 0;
    (void)algo;
    return simt_fwd_workspace_bytes(geo, tokens, dtype, layout);
}

extern "C" int nmg_spmm(const void *val, const int16_t *idx, int64_t M, int64_t K, int n, int m, int g, int dtype,
                        const void *act, int64_t ld_act, int64_t tokens, const void *bias, void *out, int64_t ld_out,
                        int layout, int algo, void *workspace, size_t workspace_bytes, void *stream) {
    Geo geo;
    int rc = make_geo(M, K, n, m, g, &geo);
    if (rc) return rc;
    if ((rc = check_common(dtype, tokens, val, idx, act, out))) return rc;
    if (n < 1) NMG_FAIL(NMG_ERR_INVALID, "n must be >= 1");
    if (layout != NMG_ACT_TOKEN_MAJOR && layout != NMG_ACT_K_MAJOR) NMG_FAIL(NMG_ERR_INVALID, "unknown activation layout %d", layout);
    const bool tm = layout == NMG_ACT_TOKEN_MAJOR;
    if (ld_act < (tm ? K : tokens)) NMG_FAIL(NMG_ERR_INVALID, "ld_act=%lld is smaller than the activation row", (long long)ld_act);
    if (ld_out < (tm ? M : tokens)) NMG_FAIL(NMG_ERR_INVALID, "ld_out=%lld is smaller than the output row", (long long)ld_out);
    if (algo == NMG_ALGO_TENSOR) NMG_FAIL(NMG_ERR_UNSUPPORTED, "tensor-core path is not available for this problem");
    if (algo != NMG_ALGO_AUTO && algo != NMG_ALGO_SIMT) NMG_FAIL(NMG_ERR_INVALID, "unknown algo %d", algo);
    return simt_fwd(geo, dtype, val, idx, act, ld_act, tokens, bias, out, ld_out, layout, workspace, workspace_bytes,
                    (cudaStream_t)stream);
}

extern "C" size_t nmg_spmm_t_workspace_bytes(int64_t M, int64_t K, int64_t tokens, int n, int m, int g, int dtype,
                                             int algo) {
    Geo geo;
    if (make_geo(M, K, n, m, g, &geo) || tokens < 1) return 0;
    (void)algo;
    return simt_bwd_workspace_bytes(geo, tokens, dtype);
}

extern "C" int nmg_spmm_t(const void *val, const int16_t *idx, int64_t M, int64_t K, int n, int m, int g, int dtype,
                          const void *dy, int64_t ld_dy, int64_t tokens, void *dx, int64_t ld_dx, int algo,
                          void *workspace, size_t workspace_bytes, void *stream) {
    Geo geo;
    int rc = make_geo(M, K, n, m, g, &geo);
    if (rc) return rc;
    if ((rc = check_common(dtype, tokens, val, idx, dy, dx))) return rc;
    if (n < 1) NMG_FAIL(NMG_ERR_INVALID, "n must be >= 1");
    if (ld_dy < M) NMG_FAIL(NMG_ERR_INVALID, "ld_dy=%lld is smaller than M", (long long)ld_dy);
    if (ld_dx < K) NMG_FAIL(NMG_ERR_INVALID, "ld_dx=%lld is smaller than K", (long long)ld_dx);
    if (algo == NMG_ALGO_TENSOR) NMG_FAIL(NMG_ERR_UNSUPPORTED, "tensor-core path is not available for this problem");
    if (algo != NMG_ALGO_AUTO && algo != NMG_ALGO_SIMT) NMG_FAIL(NMG_ERR_INVALID, "unknown algo %d", algo);
    return simt_bwd(geo, dtype, val, idx, dy, ld_dy, tokens, dx, ld_dx, workspace, workspace_bytes, (cudaStream_t)stream);
}
