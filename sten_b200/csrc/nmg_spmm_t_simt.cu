// SIMT transposed matmul  dX = dY * W  (the backward of y = x W^T with respect to x) for a grouped n:m weight.
//
// The reduction runs over the rows of W, which is the axis the n:m blocks live on, so the operand a thread
// must select dynamically is a row of dY (one of the m rows of a row-block), while the output column is
// fixed.  The kernel therefore works on a column-ordered copy of the weight (built once per call in the
// workspace by build_natural_kernel): for every row-block mb and column k it stores the column's pattern and
// its n kept values.  A warp owns KW consecutive columns; its lanes are tokens.  For every row-block the
// warp pulls the m x TT slice of dY^T from shared memory into registers once and re-uses it for all KW
// columns; the pattern of each column selects, through a warp-uniform switch over the compile-time pattern
// table, which n of those registers are multiplied.  Accumulators stay in registers over all row-blocks.
#include "nmg_spmm_simt.cuh"

namespace nmg {

// ------------------------------------------------------------------------------------------ column-ordered copy
struct NaturalParams {
    const void *val; const int16_t *idx; uint16_t *pat; void *nval;
    __nv_bfloat16 *plane[3];  // fp32 weights only, else NULL
    int64_t nb, nc, Kp;
    int n, g, cc;
};
template <typename T>
__global__ void build_natural_kernel(const NaturalParams prm) {
    const int64_t total = prm.nb * prm.nc * prm.cc;  // one thread per stored column slot
    const T *val = static_cast<const T *>(prm.val);
    T *nval = static_cast<T *>(prm.nval);
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t tile = e / prm.cc;
        const int slot = (int)(e - tile * prm.cc);
        const int64_t mb = tile % prm.nb, kc = tile / prm.nb;
        const int c = prm.idx[e];
        if (c < 0 || c >= prm.cc) continue;  // malformed index: leave the column empty
        const int64_t k = kc * prm.cc + c;
        prm.pat[mb * prm.Kp + k] = (uint16_t)(slot / prm.g);
        for (int s = 0; s < prm.n; s++) {
            const T v = val[e * prm.n + s];
            const int64_t o = (mb * prm.Kp + k) * prm.n + s;
            nval[o] = v;
            if (prm.plane[0]) {  // exact three-way split of an fp32 value into bf16 pieces
                const float f = DT<T>::to_f32(v);
                const __nv_bfloat16 hi = __float2bfloat16_rn(f);
                const float r1 = f - __bfloat162float(hi);
                const __nv_bfloat16 mid = __float2bfloat16_rn(r1);
                const __nv_bfloat16 lo = __float2bfloat16_rn(r1 - __bfloat162float(mid));
                prm.plane[0][o] = hi; prm.plane[1][o] = mid; prm.plane[2][o] = lo;
            }
        }
    }
}

// Width of the column-ordered copy: the padded weight width rounded up to the 128-column CTA tile, so every
// row segment a CTA stages is full-size and 16-byte aligned.
int64_t natural_width(const Geo &geo) { return round_up(geo.nc * geo.cc, 128); }

// Sections of the copy: pattern ids, values in the weight's dtype, and -- for fp32 weights -- three bf16 planes
// holding the exact split v = hi + mid + lo that the tensor-core kernel multiplies term by term.
NaturalLayout natural_layout(const Geo &geo, int dtype) {
    const size_t entries = (size_t)geo.nb * (size_t)natural_width(geo);
    NaturalLayout l;
    l.pat_bytes = (entries * 2 + 255) & ~(size_t)255;
    l.val_bytes = (entries * geo.n * dtype_size(dtype) + 255) & ~(size_t)255;
    l.plane_bytes = dtype == NMG_F32 ? ((entries * geo.n * 2 + 255) & ~(size_t)255) : 0;
    l.total = l.pat_bytes + l.val_bytes + 3 * l.plane_bytes;
    return l;
}

size_t natural_bytes(const Geo &geo, int dtype, size_t *pat_bytes_out) {
    const NaturalLayout l = natural_layout(geo, dtype);
    if (pat_bytes_out) *pat_bytes_out = l.pat_bytes;
    return l.total;
}

int launch_build_natural(const Geo &geo, int dtype, const void *val, const int16_t *idx, uint16_t *pat, void *nval,
                         cudaStream_t st) {
    const NaturalLayout lay = natural_layout(geo, dtype);
    NaturalParams p{val, idx, pat, nval, {nullptr, nullptr, nullptr}, geo.nb, geo.nc, natural_width(geo), geo.n, geo.g, geo.cc};
    if (lay.plane_bytes)
        for (int c = 0; c < 3; c++)
            p.plane[c] = reinterpret_cast<__nv_bfloat16 *>(static_cast<char *>(nval) + lay.val_bytes + c * lay.plane_bytes);
    const int64_t total = geo.nb * geo.nc * geo.cc;
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 64) blocks = 148 * 64;
    // every (mb, k) of the padded width is written exactly once because idx is a permutation per tile;
    // clear first so that a malformed idx leaves zeros, not stale workspace contents
    size_t pat_bytes = 0;
    const size_t all = natural_bytes(geo, dtype, &pat_bytes);
    NMG_CUDA(cudaMemsetAsync(pat, 0, pat_bytes, st));
    NMG_CUDA(cudaMemsetAsync(nval, 0, all - pat_bytes, st));
    NMG_DISPATCH_DTYPE(dtype, T, (build_natural_kernel<T><<<(unsigned)blocks, 256, 0, st>>>(p)));
    NMG_CUDA(cudaGetLastError());
    return NMG_OK;
}

// ------------------------------------------------------------------------------------------ generic kernel
struct GenBwdParams {
    const uint16_t *pat; const void *nval; const void *dy; void *dx; const int8_t *order;
    int64_t M, K, Kp, ntok, ld_dy, ld_dx, nb;
    int n, m;
};
template <typename T>
__global__ void spmm_bwd_generic_kernel(const GenBwdParams prm) {
    const int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // lanes along columns: coalesced dX stores
    const int64_t tok = blockIdx.y;
    if (k >= prm.K) return;
    const T *dy = static_cast<const T *>(prm.dy) + tok * prm.ld_dy;
    const T *nval = static_cast<const T *>(prm.nval);
    float acc = 0.f;
    for (int64_t mb = 0; mb < prm.nb; mb++) {
        const int p = prm.pat[mb * prm.Kp + k];
        for (int s = 0; s < prm.n; s++) {
            const int64_t row = mb * prm.m + prm.order[p * prm.n + s];
            if (row < prm.M) acc = fmaf(DT<T>::to_f32(nval[(mb * prm.Kp + k) * prm.n + s]), DT<T>::to_f32(dy[row]), acc);
        }
    }
    static_cast<T *>(prm.dx)[tok * prm.ld_dx + k] = DT<T>::from_f32(acc);
}

// ------------------------------------------------------------------------------------------ host side
static bool bwd_specialised(int n, int m) {
    return (n == 1 && m == 4) || (n == 2 && m == 4) || (n == 1 && m == 8) || (n == 2 && m == 8) || (n == 1 && m == 16) ||
           (n == 3 && m == 6);
}

static int bwd_rb_stage(int m) {  // rows per stage <= 64 keeps one TMA box (256-row limit) and ~32 KB of dY^T
    int rs = 64 / m;
    return rs > 0 ? rs : 1;
}

size_t simt_bwd_workspace_bytes(const Geo &geo, int64_t tokens, int dtype) {
    (void)dtype;
    return bwd_specialised(geo.n, geo.m) ? (size_t)geo.M * (size_t)round_up(tokens, 128) * 4 + 256 : 0;
}

int simt_bwd(const Geo &geo, int dtype, const uint16_t *pat, const void *nval, const void *dy, int64_t ld_dy,
             int64_t tokens, void *dx, int64_t ld_dx, void *ws, size_t ws_bytes, cudaStream_t st) {
    const size_t need = simt_bwd_workspace_bytes(geo, tokens, dtype);
    if (need && (!ws || ws_bytes < need)) NMG_FAIL(NMG_ERR_WORKSPACE, "workspace of %zu bytes required, got %zu", need, ws_bytes);
    char *base = reinterpret_cast<char *>(((uintptr_t)ws + 255) & ~(uintptr_t)255);
    int rc = NMG_OK;
    const int64_t Kp = natural_width(geo);

    if (!bwd_specialised(geo.n, geo.m)) {
        PatternTable tab;
        if ((rc = get_pattern_table(geo.n, geo.m, &tab))) return rc;
        if (tokens > 65535) NMG_FAIL(NMG_ERR_UNSUPPORTED, "generic transposed kernel handles at most 65535 tokens per call");
        GenBwdParams p{pat, nval, dy, dx, tab.order, geo.M, geo.K, Kp, tokens, ld_dy, ld_dx, geo.nb, geo.n, geo.m};
        dim3 grid((unsigned)((geo.K + 127) / 128), (unsigned)tokens);
        const ProfileEvents pe = take_profile_events();
        if (pe.start) NMG_CUDA(cudaEventRecord(pe.start, st));
        NMG_DISPATCH_DTYPE(dtype, T, (spmm_bwd_generic_kernel<T><<<grid, 128, 0, st>>>(p)));
        NMG_CUDA(cudaGetLastError());
        if (pe.stop) NMG_CUDA(cudaEventRecord(pe.stop, st));
        return NMG_OK;
    }

    float *yt = reinterpret_cast<float *>(base);
    const int64_t ld_yt = round_up(tokens, 128);
    if ((rc = launch_transpose_to_f32(dy, dtype, tokens, geo.M, ld_dy, yt, ld_yt, st))) return rc;
    const int rs = bwd_rb_stage(geo.m);
    CUtensorMap tm;
    if ((rc = encode_tmap_2d(&tm, NMG_F32, yt, (uint64_t)ld_yt, (uint64_t)geo.M, (uint64_t)ld_yt, (uint32_t)kBwdTok, (uint32_t)(rs * geo.m), 0)))
        return rc;
    int *status = nullptr;
    if ((rc = get_status_word(&status))) return rc;
    BwdParams p{pat, nval, dx, geo.M, geo.K, Kp, tokens, ld_dx, geo.nb, rs, status};
    const ProfileEvents pe = take_profile_events();
    if (pe.start) NMG_CUDA(cudaEventRecord(pe.start, st));
#define NMG_BWD_LAUNCH(N_, M_)                                                \
    if (geo.n == N_ && geo.m == M_) {                                         \
        rc = simt_bwd_launch<N_, M_>(dtype, p, tm, tokens, st);               \
        if (rc == NMG_OK && pe.stop) NMG_CUDA(cudaEventRecord(pe.stop, st));  \
        return rc;                                                            \
    }
    NMG_BWD_LAUNCH(1, 4)
    NMG_BWD_LAUNCH(2, 4)
    NMG_BWD_LAUNCH(1, 8)
    NMG_BWD_LAUNCH(2, 8)
    NMG_BWD_LAUNCH(1, 16)
    NMG_BWD_LAUNCH(3, 6)
#undef NMG_BWD_LAUNCH
    NMG_FAIL(NMG_ERR_UNSUPPORTED, "no specialised transposed kernel for %d:%d", geo.n, geo.m);
}

}  // namespace nmg
