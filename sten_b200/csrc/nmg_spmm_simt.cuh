// Declarations shared by the matmul translation units.
#pragma once
#include "nmg_common.cuh"

namespace nmg {

inline int64_t round_up(int64_t a, int64_t b) { return (a + b - 1) / b * b; }

// Activation re-layout pre-pass: src[rows][ld_src] (dtype) -> dst[cols][ld_dst] fp32, i.e. transpose + widen.
int launch_transpose_to_f32(const void *src, int dtype, int64_t rows, int64_t cols, int64_t ld_src, float *dst,
                            int64_t ld_dst, cudaStream_t st);
// Same-dtype transpose: src[rows][ld_src] -> dst[cols][ld_dst]; columns of dst beyond `rows` (up to ld_dst) are zeroed.
int launch_transpose(const void *src, int dtype, int64_t rows, int64_t cols, int64_t ld_src, void *dst, int64_t ld_dst, cudaStream_t st);
// Copy + widen without transposing: src[rows][ld_src] (dtype) -> dst[rows][ld_dst] fp32.
int launch_widen_to_f32(const void *src, int dtype, int64_t rows, int64_t cols, int64_t ld_src, float *dst,
                        int64_t ld_dst, cudaStream_t st);

// Column-order ("natural") copy of a weight: for every row-block mb and column k of the padded width Kp,
// pat[mb][k] = pattern of that column, nval[mb][k][s] = its n kept values.
struct NaturalLayout { size_t pat_bytes, val_bytes, plane_bytes, total; };
NaturalLayout natural_layout(const Geo &geo, int dtype);
int64_t natural_width(const Geo &geo);
size_t natural_bytes(const Geo &geo, int dtype, size_t *pat_bytes_out);
int launch_build_natural(const Geo &geo, int dtype, const void *val, const int16_t *idx, uint16_t *pat, void *nval,
                         cudaStream_t st);

// SIMT kernels (fp32 accumulate).  xt is the activation as [K][ld_xt] fp32 (tokens contiguous).
size_t simt_fwd_workspace_bytes(const Geo &geo, int64_t tokens, int dtype, int layout);
int simt_fwd(const Geo &geo, int dtype, const void *val, const int16_t *idx, const void *act, int64_t ld_act,
             int64_t tokens, const void *bias, void *out, int64_t ld_out, int layout, void *ws, size_t ws_bytes,
             cudaStream_t st);
// pat / nval: the column-ordered copy; the workspace only holds the fp32 transpose of dY
size_t simt_bwd_workspace_bytes(const Geo &geo, int64_t tokens, int dtype);
int simt_bwd(const Geo &geo, int dtype, const uint16_t *pat, const void *nval, const void *dy, int64_t ld_dy,
             int64_t tokens, void *dx, int64_t ld_dx, void *ws, size_t ws_bytes, cudaStream_t st);

// Tensor-core kernels.  act: [tokens][ld_act] with the reduction axis contiguous.  fp32 operands are multiplied as
// sums of bf16 pieces and need `ws` (tc_split_workspace_bytes) for the split activation.  Two variants share the
// entry point tc_matmul: the fused kernel (nmg_spmm_tc.cu) expands the column-ordered copy (pat / nval) tile by tile
// inside the matmul; the two-pass variant (nmg_gemm_tc.cu, `dense` = true) first expands (val, idx) into a dense 16-bit
// matrix in `ws` (tc_dense_workspace_bytes, after the split activation) and multiplies that.  tc_use_dense is the
// policy: two passes from 1280 tokens on (256 for fp32), and for every (n, m) the fused kernel has no instantiation for.
// What follows the product: out = activation(product + bias) + residual.  The two-pass tensor-core matmul applies it in its
// epilogue; every other kernel is followed by one elementwise pass (launch_epilogue).
struct Epilogue {
    int act = NMG_EPI_NONE;
    const void *residual = nullptr;  // same orientation as the output
    int64_t ld_res = 0;
    bool any() const { return act != NMG_EPI_NONE || residual != nullptr; }
};
int launch_epilogue(int dtype, void *out, int64_t rows, int64_t cols, int64_t ld_out, const Epilogue &epi, cudaStream_t st);
bool tc_dense_uses_pair(const Geo &geo, int dtype, bool transposed);

bool tc_supported(const Geo &geo, int dtype);        // fused kernel
bool tc_dense_supported(const Geo &geo, int dtype);  // two-pass variant
bool tc_use_dense(const Geo &geo, int dtype, int64_t tokens);
size_t tc_split_workspace_bytes(const Geo &geo, int dtype, bool transposed, int64_t tokens);
size_t tc_dense_workspace_bytes(const Geo &geo, int dtype, bool transposed);
// fused kernel with few output tiles: the reduction axis is cut over tc_ksplit CTAs per tile, fp32 partial tiles in `ws`
int tc_ksplit(const Geo &geo, int dtype, bool transposed, int64_t tokens);
size_t tc_ksplit_workspace_bytes(const Geo &geo, int dtype, bool transposed, int64_t tokens);
// outs / n_outs: the result goes to every listed buffer (same shape and pitch); more than one needs `dense`.  mc_out, when
// not NULL, is an NVSwitch multicast address that maps onto all of them: full 16-byte chunks are then stored once.
int tc_matmul(const Geo &geo, int dtype, bool transposed, bool dense, const void *val, const int16_t *idx, const uint16_t *pat,
              const void *nval, const void *act, int64_t ld_act, int64_t tokens, const void *bias, void *const *outs, int n_outs,
              void *mc_out, int64_t ld_out, int out_token_major, void *ws, size_t ws_bytes, cudaStream_t st, const Epilogue &epi = Epilogue());
int tc_dense_matmul(const Geo &geo, int dtype, bool transposed, const void *val, const int16_t *idx, const CUtensorMap *act_maps,
                    int64_t tokens, const void *bias, void *const *outs, int n_outs, void *mc_out, int64_t ld_out, int out_token_major,
                    void *ws, size_t ws_bytes, cudaStream_t st, const Epilogue &epi);

// Structured-sparse tensor-core path of the transposed product (nmg_gemm_sp.cu): tcgen05.mma.sp on W^T compressed along
// the reduction axis (the weight's rows).  16-bit weights with n <= 2 and m in {4, 8, 16, 32, 64}; taken from the token
// count at which the two-pass variant is taken (the compression pass is per call, like the dense expansion).
bool tc_sp_supported(const Geo &geo, int dtype);
size_t tc_sp_copy_bytes(const Geo &geo);  // compressed transposed copy: values of W^T (M * K bytes) + metadata (M * K / 8)
int tc_sp_pack(const Geo &geo, int dtype, const void *val, const int16_t *idx, void *buf, size_t buf_bytes, cudaStream_t st);
int tc_sp_matmul_t(const Geo &geo, int dtype, const void *sp_copy, const void *dy, int64_t ld_dy, int64_t tokens, void *dx, int64_t ld_dx,
                   cudaStream_t st);

// The two halves of the two-pass variant on their own: a caller may keep the expanded weight across calls (opt-in: it
// trades the format's memory saving for skipping the expansion pass of every call).
int tc_dense_expand(const Geo &geo, int dtype, bool transposed, const void *val, const int16_t *idx, char *dense, cudaStream_t st);
int tc_dense_gemm(int64_t rows, int64_t red, int dtype, bool pair, const char *dense, const CUtensorMap *act_maps, int64_t tokens,
                  const void *bias, void *const *outs, int n_outs, void *mc_out, int64_t ld_out, int out_token_major, cudaStream_t st,
                  const Epilogue &epi);

// ---- specialised forward kernel: parameters, shared-memory plan, per-(n, m) launchers
struct FwdParams {
    const void *val;
    const int16_t *idx;
    const void *bias;
    void *out;
    int64_t M, K, ntok, ld_out;
    int64_t nb, nc;
    int g, cc;
    int box_rows, nbox;  // TMA boxes per chunk: nbox boxes of box_rows activation rows
    int stages;
    int *status;
};

constexpr int kWarps = 8;

struct FwdSmemPlan {
    size_t x_bytes, v_bytes, i_bytes, stage_bytes, total;
};
__host__ __device__ inline FwdSmemPlan fwd_smem_plan(int cc, int n, int rbc, int tokc, int nbox, int box_rows, size_t es, int stages) {
    FwdSmemPlan p;
    p.x_bytes = (size_t)nbox * box_rows * tokc * 4;
    p.v_bytes = (((size_t)rbc * cc * n * es + 32) + 127) & ~(size_t)127;
    p.i_bytes = (((size_t)rbc * cc * 2 + 32) + 127) & ~(size_t)127;
    p.stage_bytes = p.x_bytes + p.v_bytes + p.i_bytes;
    p.total = p.stage_bytes * stages + 128 /*barriers*/ + 128 /*alignment slack*/;
    return p;
}

// Which (n, m) have a specialised forward kernel, and the tile configuration chosen for a geometry.
struct FwdChoice { int tt, stages; };
bool simt_fwd_specialised(int n, int m);
bool choose_fwd(const Geo &geo, size_t es, FwdChoice *c, int *box_rows, int *nbox);

template <int N_, int M_>
int simt_fwd_launch(int dtype, int tt, const FwdParams &p, const CUtensorMap &tm, int rbc, size_t smem, bool token_major,
                    int64_t tokens, cudaStream_t st);

// ---- specialised transposed kernel: parameters, shared-memory plan, per-(n, m) launchers
struct BwdParams {
    const uint16_t *pat;  // [nb][Kp]
    const void *nval;     // [nb][Kp][n]
    void *dx;
    int64_t M, K, Kp, ntok, ld_dx, nb;
    int rb_stage;    // row-blocks per pipeline stage
    int *status;
};

constexpr int kBwdWarps = 8;
constexpr int kKW = 16;                      // columns per warp
constexpr int kColsCta = kBwdWarps * kKW;    // 128 columns per CTA
constexpr int kBwdTT = 4;
constexpr int kBwdTok = 32 * kBwdTT;         // 128 tokens per CTA

struct BwdSmemPlan { size_t y_bytes, p_bytes, v_bytes, stage_bytes, total; };
__host__ __device__ inline BwdSmemPlan bwd_smem_plan(int m, int n, int rb_stage, size_t es) {
    BwdSmemPlan p;
    p.y_bytes = (size_t)rb_stage * m * kBwdTok * 4;
    p.p_bytes = ((size_t)rb_stage * kColsCta * 2 + 127) & ~(size_t)127;
    p.v_bytes = ((size_t)rb_stage * kColsCta * n * es + 127) & ~(size_t)127;
    p.stage_bytes = p.y_bytes + p.p_bytes + p.v_bytes;
    p.total = 2 * p.stage_bytes + 256;
    return p;
}

template <int N_, int M_>
int simt_bwd_launch(int dtype, const BwdParams &p, const CUtensorMap &tm, int64_t tokens, cudaStream_t st);

}  // namespace nmg
