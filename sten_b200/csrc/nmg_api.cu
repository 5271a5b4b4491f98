// C-ABI entry points of the matmul and of the packed (column-ordered) weight copy: argument validation, choice of
// kernel family, workspace carving.
#include "nmg_spmm_simt.cuh"

using namespace nmg;

static int check_common(int dtype, int64_t tokens, const void *a, const void *b, const void *c, const void *d) {
    if (dtype != NMG_F32 && dtype != NMG_F16 && dtype != NMG_BF16)
        NMG_FAIL(NMG_ERR_INVALID, "dtype must be NMG_F32, NMG_F16 or NMG_BF16, got %d", dtype);
    if (tokens < 1) NMG_FAIL(NMG_ERR_INVALID, "tokens must be positive, got %lld", (long long)tokens);
    if (!a || !b || !c || !d) NMG_FAIL(NMG_ERR_INVALID, "NULL operand pointer");
    return NMG_OK;
}

static char *align256(void *p) { return reinterpret_cast<char *>(((uintptr_t)p + 255) & ~(uintptr_t)255); }

// The tensor-core kernel reads the activation through a TMA descriptor: 16-bit dtype, reduction axis contiguous,
// 16-byte aligned base and row pitch.
static bool tensor_ok(const Geo &geo, int dtype, const void *act, int64_t ld_act) {
    if (!tc_supported(geo, dtype) && !tc_dense_supported(geo, dtype)) return false;
    if (dtype == NMG_F32) return true;  // fp32 activations are re-laid out into aligned bf16 planes first
    return (((uintptr_t)act) & 15) == 0 && (ld_act % 8) == 0;
}

extern "C" size_t nmg_packed_bytes(int64_t M, int64_t K, int n, int m, int g, int dtype) {
    Geo geo;
    if (make_geo(M, K, n, m, g, &geo) || n < 1) return 0;
    return natural_bytes(geo, dtype, nullptr) + 256;
}

extern "C" int nmg_pack(const void *val, const int16_t *idx, int64_t M, int64_t K, int n, int m, int g, int dtype,
                        void *packed, size_t packed_bytes, void *stream) {
    Geo geo;
    int rc = make_geo(M, K, n, m, g, &geo);
    if (rc) return rc;
    if ((rc = check_common(dtype, 1, val, idx, packed, packed))) return rc;
    if (n < 1) NMG_FAIL(NMG_ERR_INVALID, "n must be >= 1");
    size_t pat_bytes = 0;
    const size_t need = natural_bytes(geo, dtype, &pat_bytes) + 256;
    if (packed_bytes < need) NMG_FAIL(NMG_ERR_WORKSPACE, "packed buffer of %zu bytes required, got %zu", need, packed_bytes);
    char *base = align256(packed);
    return launch_build_natural(geo, dtype, val, idx, reinterpret_cast<uint16_t *>(base), base + pat_bytes, (cudaStream_t)stream);
}

// Resolve the column-ordered copy: the caller's, or one built at the front of the workspace.  Advances *ws.
static int resolve_packed(const Geo &geo, int dtype, const void *val, const int16_t *idx, const void *packed, char **ws,
                          size_t *ws_left, const uint16_t **pat, const void **nval, cudaStream_t st) {
    size_t pat_bytes = 0;
    const size_t nat = natural_bytes(geo, dtype, &pat_bytes);
    if (packed) {
        char *base = align256(const_cast<void *>(packed));
        *pat = reinterpret_cast<const uint16_t *>(base);
        *nval = base + pat_bytes;
        return NMG_OK;
    }
    if (!*ws || *ws_left < nat + 256) NMG_FAIL(NMG_ERR_WORKSPACE, "workspace too small for the column-ordered weight copy (%zu bytes)", nat + 256);
    char *base = align256(*ws);
    *pat = reinterpret_cast<const uint16_t *>(base);
    *nval = base + pat_bytes;
    *ws_left -= (size_t)(base + nat - *ws);
    *ws = base + nat;
    return launch_build_natural(geo, dtype, val, idx, reinterpret_cast<uint16_t *>(base), base + pat_bytes, st);
}

// K-major activations (B[K][tokens], the torch.mm orientation) reach the tensor cores through one same-dtype transpose
// into the workspace: X[tokens][round_up(K, 8)], after which the call is the token-major one with row-major output.
static size_t kmajor_transpose_bytes(const Geo &geo, int dtype, int64_t tokens) {
    return (size_t)tokens * (size_t)round_up(geo.K, 8) * dtype_size(dtype) + 512;
}

extern "C" size_t nmg_spmm_workspace_bytes(int64_t M, int64_t K, int64_t tokens, int n, int m, int g, int dtype,
                                           int layout, int algo, int have_packed) {
    Geo geo;
    if (make_geo(M, K, n, m, g, &geo) || tokens < 1 || n < 1) return 0;
    size_t simt = simt_fwd_workspace_bytes(geo, tokens, dtype, layout);
    size_t tensor = 0;
    if (algo == NMG_ALGO_TENSOR_DENSE) algo = NMG_ALGO_TENSOR;
    if (algo != NMG_ALGO_SIMT && (tc_supported(geo, dtype) || tc_dense_supported(geo, dtype)))
        tensor = (tc_use_dense(geo, dtype, tokens) ? tc_dense_workspace_bytes(geo, dtype, false)
                                                   : (have_packed ? 0 : natural_bytes(geo, dtype, nullptr) + 512) +
                                                         tc_ksplit_workspace_bytes(geo, dtype, false, tokens)) +
                 tc_split_workspace_bytes(geo, dtype, false, tokens) + (layout == NMG_ACT_K_MAJOR ? kmajor_transpose_bytes(geo, dtype, tokens) : 0);
    if (algo == NMG_ALGO_TENSOR) return tensor;
    return simt > tensor ? simt : tensor;  // AUTO may take either path depending on operand alignment
}

static int spmm_impl(const void *val, const int16_t *idx, const void *packed, int64_t M, int64_t K, int n, int m, int g, int dtype,
                     const void *act, int64_t ld_act, int64_t tokens, const void *bias, void *const *outs, int n_outs, int64_t ld_out,
                     int layout, int algo, void *workspace, size_t workspace_bytes, void *stream, bool force_dense = false, void *mc_out = nullptr,
                     const Epilogue &epi = Epilogue()) {
    Geo geo;
    int rc = make_geo(M, K, n, m, g, &geo);
    if (rc) return rc;
    void *out = outs[0];
    if ((rc = check_common(dtype, tokens, val, idx, act, out))) return rc;
    if (n < 1) NMG_FAIL(NMG_ERR_INVALID, "n must be >= 1");
    if (layout != NMG_ACT_TOKEN_MAJOR && layout != NMG_ACT_K_MAJOR && layout != NMG_ACT_TOKEN_MAJOR_OUT_ROWS)
        NMG_FAIL(NMG_ERR_INVALID, "unknown activation layout %d", layout);
    const bool tm = layout != NMG_ACT_K_MAJOR;               // activation rows are tokens
    const bool out_tm = layout == NMG_ACT_TOKEN_MAJOR;       // output rows are tokens
    if (ld_act < (tm ? K : tokens)) NMG_FAIL(NMG_ERR_INVALID, "ld_act=%lld is smaller than the activation row", (long long)ld_act);
    if (ld_out < (out_tm ? M : tokens)) NMG_FAIL(NMG_ERR_INVALID, "ld_out=%lld is smaller than the output row", (long long)ld_out);
    if (algo != NMG_ALGO_AUTO && algo != NMG_ALGO_SIMT && algo != NMG_ALGO_TENSOR && algo != NMG_ALGO_TENSOR_DENSE)
        NMG_FAIL(NMG_ERR_INVALID, "unknown algo %d", algo);
    if (algo == NMG_ALGO_TENSOR_DENSE) algo = NMG_ALGO_TENSOR;  // the forward product has no structured-sparse variant
    cudaStream_t st = (cudaStream_t)stream;
    // K-major activations take the tensor cores when the weight is large enough to pay for the transpose pre-pass
    const bool kmajor_tensor = !tm && n_outs == 1 && (tc_supported(geo, dtype) || tc_dense_supported(geo, dtype)) &&
                               (algo == NMG_ALGO_TENSOR || (algo == NMG_ALGO_AUTO && M >= 64 && tokens >= 64));
    if (kmajor_tensor) {
        const size_t need = kmajor_transpose_bytes(geo, dtype, tokens);
        if (!workspace || workspace_bytes < need) NMG_FAIL(NMG_ERR_WORKSPACE, "workspace of %zu bytes required for the transposed activation, got %zu", need, workspace_bytes);
        char *xt = align256(workspace);
        const int64_t ld_xt = round_up(K, 8);
        if ((rc = launch_transpose(act, dtype, K, tokens, ld_act, xt, ld_xt, st))) return rc;
        char *rest = xt + (size_t)tokens * ld_xt * dtype_size(dtype);
        const size_t used = (size_t)(rest - static_cast<char *>(workspace));
        return spmm_impl(val, idx, packed, M, K, n, m, g, dtype, xt, ld_xt, tokens, bias, outs, n_outs, ld_out, NMG_ACT_TOKEN_MAJOR_OUT_ROWS,
                         NMG_ALGO_TENSOR, rest, workspace_bytes - used, stream, force_dense, mc_out, epi);
    }
    const bool can_tensor = tm && tensor_ok(geo, dtype, act, ld_act);
    if (algo == NMG_ALGO_TENSOR && !can_tensor)
        NMG_FAIL(NMG_ERR_UNSUPPORTED, "tensor-core path needs activation rows that are 16-byte aligned (16-bit dtypes) and a chunk that fits shared memory");
    // AUTO: tensor cores whenever the operands allow it and the weight has at least 64 rows, at every token count (measured
    // at 16 tokens on a 4096^2 bf16 weight: 0.05 ms against 0.71 ms on the SIMT kernel, which is built for wide token
    // tiles); unsupported layouts / alignments and tiny weights stay on the SIMT kernels.  fp32 on tensor cores means exact bf16 splitting with
    // promoted accumulation (measured relative error 3.5e-6, independent of K); NMG_ALGO_SIMT keeps plain fp32 FMAs.
    if (algo == NMG_ALGO_TENSOR || (algo == NMG_ALGO_AUTO && can_tensor && M >= 64)) {
        char *ws = static_cast<char *>(workspace);
        size_t left = workspace_bytes;
        const uint16_t *pat = nullptr;
        const void *nval = nullptr;
        const bool dense = force_dense || tc_use_dense(geo, dtype, tokens);
        if (!dense && (rc = resolve_packed(geo, dtype, val, idx, packed, &ws, &left, &pat, &nval, st))) return rc;
        return tc_matmul(geo, dtype, false, dense, val, idx, pat, nval, act, ld_act, tokens, bias, outs, n_outs, mc_out, ld_out, out_tm ? 1 : 0, ws, left, st, epi);
    }
    if (n_outs > 1) NMG_FAIL(NMG_ERR_UNSUPPORTED, "several output buffers need the tensor-core path (aligned token-major activations, >= 64 tokens and rows)");
    if ((rc = simt_fwd(geo, dtype, val, idx, act, ld_act, tokens, bias, out, ld_out, layout, workspace, workspace_bytes, st))) return rc;
    return out_tm ? launch_epilogue(dtype, out, tokens, M, ld_out, epi, st) : launch_epilogue(dtype, out, M, tokens, ld_out, epi, st);
}

extern "C" int nmg_spmm(const void *val, const int16_t *idx, const void *packed, int64_t M, int64_t K, int n, int m,
                        int g, int dtype, const void *act, int64_t ld_act, int64_t tokens, const void *bias, void *out,
                        int64_t ld_out, int layout, int algo, void *workspace, size_t workspace_bytes, void *stream) {
    void *outs[1] = {out};
    return spmm_impl(val, idx, packed, M, K, n, m, g, dtype, act, ld_act, tokens, bias, outs, 1, ld_out, layout, algo, workspace,
                     workspace_bytes, stream);
}

extern "C" int nmg_spmm_fused(const void *val, const int16_t *idx, const void *packed, int64_t M, int64_t K, int n, int m, int g,
                              int dtype, const void *act, int64_t ld_act, int64_t tokens, const void *bias, int activation,
                              const void *residual, int64_t ld_res, void *out, int64_t ld_out, int layout, int algo, void *workspace,
                              size_t workspace_bytes, void *stream) {
    if (activation != NMG_EPI_NONE && activation != NMG_EPI_GELU) NMG_FAIL(NMG_ERR_INVALID, "unknown activation %d", activation);
    const bool out_tm = layout == NMG_ACT_TOKEN_MAJOR;
    if (residual && ld_res < (out_tm ? M : tokens)) NMG_FAIL(NMG_ERR_INVALID, "ld_res=%lld is smaller than the output row", (long long)ld_res);
    Epilogue epi;
    epi.act = activation; epi.residual = residual; epi.ld_res = ld_res;
    void *outs[1] = {out};
    return spmm_impl(val, idx, packed, M, K, n, m, g, dtype, act, ld_act, tokens, bias, outs, 1, ld_out, layout, algo, workspace,
                     workspace_bytes, stream, false, nullptr, epi);
}

extern "C" int nmg_spmm_replicated(const void *val, const int16_t *idx, int64_t M, int64_t K, int n, int m, int g, int dtype,
                                   const void *act, int64_t ld_act, int64_t tokens, const void *bias, void *const *outs, int n_outs,
                                   void *multicast_out, int64_t ld_out, void *workspace, size_t workspace_bytes, void *stream) {
    if (!outs || n_outs < 1 || n_outs > 8) NMG_FAIL(NMG_ERR_INVALID, "between 1 and 8 output buffers, got %d", n_outs);
    for (int d = 0; d < n_outs; d++)
        if (!outs[d]) NMG_FAIL(NMG_ERR_INVALID, "output buffer %d is NULL", d);
    Geo geo;
    int rc = make_geo(M, K, n, m, g, &geo);
    if (rc) return rc;
    if (!tc_dense_supported(geo, dtype))
        NMG_FAIL(NMG_ERR_UNSUPPORTED, "the replicated-output matmul runs on the two-pass tensor-core variant, which this chunk size does not fit");
    return spmm_impl(val, idx, nullptr, M, K, n, m, g, dtype, act, ld_act, tokens, bias, outs, n_outs, ld_out, NMG_ACT_TOKEN_MAJOR_OUT_ROWS,
                     NMG_ALGO_TENSOR, workspace, workspace_bytes, stream, true, multicast_out);
}

extern "C" size_t nmg_spmm_replicated_workspace_bytes(int64_t M, int64_t K, int64_t tokens, int n, int m, int g, int dtype) {
    Geo geo;
    if (make_geo(M, K, n, m, g, &geo) || tokens < 1 || n < 1 || !tc_dense_supported(geo, dtype)) return 0;
    return tc_dense_workspace_bytes(geo, dtype, false) + tc_split_workspace_bytes(geo, dtype, false, tokens);
}

extern "C" int nmg_spmm_uses_packed(int64_t M, int64_t K, int64_t tokens, int n, int m, int g, int dtype, int layout,
                                    int algo, int transposed) {
    Geo geo;
    if (make_geo(M, K, n, m, g, &geo) || tokens < 1 || n < 1) return 0;
    const bool any_tc = tc_supported(geo, dtype) || tc_dense_supported(geo, dtype);
    const bool wants = algo == NMG_ALGO_TENSOR || algo == NMG_ALGO_TENSOR_DENSE || (algo == NMG_ALGO_AUTO && (transposed ? K : M) >= 64);
    const bool tensor = any_tc && wants && (transposed || layout != NMG_ACT_K_MAJOR || tokens >= 64 || algo == NMG_ALGO_TENSOR);
    if (tensor) return tc_use_dense(geo, dtype, tokens) ? 0 : 1;
    return transposed ? 1 : 0;  // SIMT: the transposed kernel reads the packed copy, the forward kernel val / idx
}

// Whether nmg_spmm_t takes the structured-sparse tensor-core path: a supported 16-bit weight, enough tokens for the
// two-pass regime, and the caller did not ask for the dense-rate kernels.
static bool use_sp(const Geo &geo, int dtype, int64_t tokens, int algo) {
    return algo != NMG_ALGO_SIMT && algo != NMG_ALGO_TENSOR_DENSE && tc_sp_supported(geo, dtype) && tc_use_dense(geo, dtype, tokens);
}

extern "C" size_t nmg_spmm_t_workspace_bytes(int64_t M, int64_t K, int64_t tokens, int n, int m, int g, int dtype,
                                             int algo, int have_packed) {
    Geo geo;
    if (make_geo(M, K, n, m, g, &geo) || tokens < 1 || n < 1) return 0;
    const size_t pack = have_packed ? 0 : natural_bytes(geo, dtype, nullptr) + 512;
    const size_t simt = algo != NMG_ALGO_TENSOR ? pack + simt_bwd_workspace_bytes(geo, tokens, dtype) + 256 : 0;
    size_t tensor = 0;
    if (algo != NMG_ALGO_SIMT && (tc_supported(geo, dtype) || tc_dense_supported(geo, dtype)))
        tensor = (tc_use_dense(geo, dtype, tokens) ? tc_dense_workspace_bytes(geo, dtype, true)
                                                   : pack + tc_ksplit_workspace_bytes(geo, dtype, true, tokens)) +
                 tc_split_workspace_bytes(geo, dtype, true, tokens);
    if (use_sp(geo, dtype, tokens, algo) && tc_sp_copy_bytes(geo) + 256 > tensor) tensor = tc_sp_copy_bytes(geo) + 256;
    return simt > tensor ? simt : tensor;
}

extern "C" int nmg_spmm_t(const void *val, const int16_t *idx, const void *packed, int64_t M, int64_t K, int n, int m,
                          int g, int dtype, const void *dy, int64_t ld_dy, int64_t tokens, void *dx, int64_t ld_dx,
                          int algo, void *workspace, size_t workspace_bytes, void *stream) {
    Geo geo;
    int rc = make_geo(M, K, n, m, g, &geo);
    if (rc) return rc;
    if ((rc = check_common(dtype, tokens, val, idx, dy, dx))) return rc;
    if (n < 1) NMG_FAIL(NMG_ERR_INVALID, "n must be >= 1");
    if (ld_dy < M) NMG_FAIL(NMG_ERR_INVALID, "ld_dy=%lld is smaller than M", (long long)ld_dy);
    if (ld_dx < K) NMG_FAIL(NMG_ERR_INVALID, "ld_dx=%lld is smaller than K", (long long)ld_dx);
    if (algo != NMG_ALGO_AUTO && algo != NMG_ALGO_SIMT && algo != NMG_ALGO_TENSOR && algo != NMG_ALGO_TENSOR_DENSE)
        NMG_FAIL(NMG_ERR_INVALID, "unknown algo %d", algo);
    cudaStream_t st = (cudaStream_t)stream;
    const bool can_tensor = tensor_ok(geo, dtype, dy, ld_dy);
    if ((algo == NMG_ALGO_TENSOR || algo == NMG_ALGO_TENSOR_DENSE) && !can_tensor)
        NMG_FAIL(NMG_ERR_UNSUPPORTED, "tensor-core path needs gradient rows that are 16-byte aligned (16-bit dtypes) and a chunk that fits shared memory");
    char *ws = static_cast<char *>(workspace);
    size_t left = workspace_bytes;
    const uint16_t *pat = nullptr;
    const void *nval = nullptr;
    const bool tensor = algo == NMG_ALGO_TENSOR || algo == NMG_ALGO_TENSOR_DENSE || (algo == NMG_ALGO_AUTO && can_tensor && K >= 64);
    // The rows of W are the reduction axis here, so the n:m structure is one the tensor cores can skip: structured-sparse
    // MMA at twice the dense rate (16-bit weights, n <= 2, m a power of two >= 4).
    if (tensor && use_sp(geo, dtype, tokens, algo)) {
        const size_t need = tc_sp_copy_bytes(geo);
        char *buf = align256(workspace);
        if (!workspace || workspace_bytes < need + 256) NMG_FAIL(NMG_ERR_WORKSPACE, "workspace of %zu bytes required for the compressed transposed weight, got %zu", need + 256, workspace_bytes);
        const ProfileEvents pe = take_profile_events();
        if (pe.start) NMG_CUDA(cudaEventRecord(pe.start, st));
        if ((rc = tc_sp_pack(geo, dtype, val, idx, buf, need, st))) return rc;
        rc = tc_sp_matmul_t(geo, dtype, buf, dy, ld_dy, tokens, dx, ld_dx, st);
        if (rc == NMG_OK && pe.stop) NMG_CUDA(cudaEventRecord(pe.stop, st));
        return rc;
    }
    const bool dense = tensor && tc_use_dense(geo, dtype, tokens);
    if (!dense && (rc = resolve_packed(geo, dtype, val, idx, packed, &ws, &left, &pat, &nval, st))) return rc;
    void *dxs[1] = {dx};
    if (tensor) return tc_matmul(geo, dtype, true, dense, val, idx, pat, nval, dy, ld_dy, tokens, nullptr, dxs, 1, nullptr, ld_dx, 1, ws, left, st);
    return simt_bwd(geo, dtype, pat, nval, dy, ld_dy, tokens, dx, ld_dx, ws, left, st);
}

// ---- compressed transposed copy ("sp24") kept by the caller ---------------------------------------------------------
extern "C" size_t nmg_sp24_bytes(int64_t M, int64_t K, int n, int m, int g, int dtype) {
    Geo geo;
    if (make_geo(M, K, n, m, g, &geo) || !tc_sp_supported(geo, dtype)) return 0;
    return tc_sp_copy_bytes(geo);
}

extern "C" int nmg_pack_sp24(const void *val, const int16_t *idx, int64_t M, int64_t K, int n, int m, int g, int dtype, void *sp24,
                             size_t sp24_bytes, void *stream) {
    Geo geo;
    int rc = make_geo(M, K, n, m, g, &geo);
    if (rc) return rc;
    if ((rc = check_common(dtype, 1, val, idx, sp24, sp24))) return rc;
    return tc_sp_pack(geo, dtype, val, idx, sp24, sp24_bytes, (cudaStream_t)stream);
}

extern "C" int nmg_spmm_t_sp24(const void *sp24, int64_t M, int64_t K, int n, int m, int g, int dtype, const void *dy, int64_t ld_dy,
                               int64_t tokens, void *dx, int64_t ld_dx, void *stream) {
    Geo geo;
    int rc = make_geo(M, K, n, m, g, &geo);
    if (rc) return rc;
    if ((rc = check_common(dtype, tokens, sp24, sp24, dy, dx))) return rc;
    if (ld_dy < M) NMG_FAIL(NMG_ERR_INVALID, "ld_dy=%lld is smaller than M", (long long)ld_dy);
    if (ld_dx < K) NMG_FAIL(NMG_ERR_INVALID, "ld_dx=%lld is smaller than K", (long long)ld_dx);
    cudaStream_t st = (cudaStream_t)stream;
    const ProfileEvents pe = take_profile_events();
    if (pe.start) NMG_CUDA(cudaEventRecord(pe.start, st));
    rc = tc_sp_matmul_t(geo, dtype, sp24, dy, ld_dy, tokens, dx, ld_dx, st);
    if (rc == NMG_OK && pe.stop) NMG_CUDA(cudaEventRecord(pe.stop, st));
    return rc;
}

// ---- expanded weight kept by the caller (opt-in) ----------------------------------------------------------------------
extern "C" size_t nmg_expanded_bytes(int64_t M, int64_t K, int n, int m, int g, int dtype) {
    Geo geo;
    if (make_geo(M, K, n, m, g, &geo) || (dtype != NMG_F16 && dtype != NMG_BF16) || !tc_dense_supported(geo, dtype)) return 0;
    return tc_dense_workspace_bytes(geo, dtype, false);
}

extern "C" int nmg_expand(const void *val, const int16_t *idx, int64_t M, int64_t K, int n, int m, int g, int dtype, void *expanded,
                          size_t expanded_bytes, void *stream) {
    Geo geo;
    int rc = make_geo(M, K, n, m, g, &geo);
    if (rc) return rc;
    if ((rc = check_common(dtype, 1, val, idx, expanded, expanded))) return rc;
    if (dtype == NMG_F32 || !tc_dense_supported(geo, dtype)) NMG_FAIL(NMG_ERR_UNSUPPORTED, "the expanded copy exists for 16-bit weights whose chunk fits shared memory");
    if (expanded_bytes < tc_dense_workspace_bytes(geo, dtype, false) || (reinterpret_cast<uintptr_t>(expanded) & 255))
        NMG_FAIL(NMG_ERR_WORKSPACE, "the expanded copy needs %zu bytes, 256-byte aligned", tc_dense_workspace_bytes(geo, dtype, false));
    return tc_dense_expand(geo, dtype, false, val, idx, static_cast<char *>(expanded), (cudaStream_t)stream);
}

extern "C" int nmg_spmm_expanded(const void *expanded, int64_t M, int64_t K, int dtype, const void *act, int64_t ld_act, int64_t tokens,
                                 const void *bias, int activation, const void *residual, int64_t ld_res, void *out, int64_t ld_out,
                                 int layout, void *stream) {
    int rc;
    if ((rc = check_common(dtype, tokens, expanded, expanded, act, out))) return rc;
    if (dtype == NMG_F32) NMG_FAIL(NMG_ERR_UNSUPPORTED, "the expanded copy exists for 16-bit weights");
    if (M < 1 || K < 1) NMG_FAIL(NMG_ERR_INVALID, "weight shape must be positive");
    if (layout != NMG_ACT_TOKEN_MAJOR && layout != NMG_ACT_TOKEN_MAJOR_OUT_ROWS) NMG_FAIL(NMG_ERR_UNSUPPORTED, "token-major activations only");
    if (activation != NMG_EPI_NONE && activation != NMG_EPI_GELU) NMG_FAIL(NMG_ERR_INVALID, "unknown activation %d", activation);
    const bool out_tm = layout == NMG_ACT_TOKEN_MAJOR;
    if (ld_act < K || ld_out < (out_tm ? M : tokens) || (residual && ld_res < (out_tm ? M : tokens))) NMG_FAIL(NMG_ERR_INVALID, "leading dimension smaller than the row");
    if ((reinterpret_cast<uintptr_t>(expanded) & 255) || (reinterpret_cast<uintptr_t>(act) & 15) || (ld_act % 8))
        NMG_FAIL(NMG_ERR_UNSUPPORTED, "the expanded copy must be 256-byte aligned and the activation rows 16-byte aligned");
    const bool pair = M > 128;
    CUtensorMap tm[3];
    if ((rc = encode_tmap_2d(&tm[0], dtype, act, (uint64_t)K, (uint64_t)tokens, (uint64_t)ld_act, 64, pair ? 128 : 256, 1))) return rc;
    tm[1] = tm[0];
    tm[2] = tm[0];
    Epilogue epi;
    epi.act = activation; epi.residual = residual; epi.ld_res = ld_res;
    void *outs[1] = {out};
    cudaStream_t st = (cudaStream_t)stream;
    const ProfileEvents pe = take_profile_events();
    if (pe.start) NMG_CUDA(cudaEventRecord(pe.start, st));
    rc = tc_dense_gemm(M, K, dtype, pair, static_cast<const char *>(expanded), tm, tokens, bias, outs, 1, nullptr, ld_out, out_tm ? 1 : 0, st, epi);
    if (rc == NMG_OK && pe.stop) NMG_CUDA(cudaEventRecord(pe.stop, st));
    return rc;
}
