// SIMT forward matmul  out = act * W^T  for a grouped n:m weight, any dtype, fp32 accumulation.
//
// Work decomposition: a CTA owns 32*TT tokens and 8*RBW row-blocks and walks all column chunks.  Per chunk the
// activation tile [cc columns][32*TT tokens] (fp32, tokens contiguous) arrives by TMA into shared memory, and the
// val / idx slabs of the CTA's row-blocks arrive by cp.async; both are double buffered.  A warp owns RBW
// row-blocks; its lanes are tokens.  Because the kernel is specialised on (n, m) the pattern table is a
// compile-time constant and the walk over the C pattern groups is unrolled: the rows a group writes are
// known statically, so the n*TT products of a column go straight into per-row register accumulators that
// live across the whole reduction.  Only non-zeros are multiplied; there are no atomics and the summation
// order is fixed.
#include "nmg_spmm_simt.cuh"

namespace nmg {

// ------------------------------------------------------------------------------------------ re-layout pre-passes
template <typename T>
__global__ void transpose_to_f32_kernel(const T *__restrict__ src, int64_t rows, int64_t cols, int64_t ld_src,
                                        float *__restrict__ dst, int64_t ld_dst) {
    __shared__ float tile[32][33];
    const int64_t c0 = (int64_t)blockIdx.x * 32, r0 = (int64_t)blockIdx.y * 32;
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int64_t r = r0 + i, c = c0 + threadIdx.x;
        tile[i][threadIdx.x] = (r < rows && c < cols) ? DT<T>::to_f32(src[r * ld_src + c]) : 0.f;
    }
    __syncthreads();
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int64_t c = c0 + i, r = r0 + threadIdx.x;
        if (c < cols && r < ld_dst) dst[c * ld_dst + r] = tile[threadIdx.x][i];  // pad columns (r >= rows) get 0
    }
}

template <typename T>
__global__ void widen_to_f32_kernel(const T *__restrict__ src, int64_t rows, int64_t cols, int64_t ld_src,
                                    float *__restrict__ dst, int64_t ld_dst) {
    const int64_t r = blockIdx.y;
    for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < ld_dst; c += (int64_t)gridDim.x * blockDim.x)
        dst[r * ld_dst + c] = c < cols ? DT<T>::to_f32(src[r * ld_src + c]) : 0.f;
}

int launch_transpose_to_f32(const void *src, int dtype, int64_t rows, int64_t cols, int64_t ld_src, float *dst,
                            int64_t ld_dst, cudaStream_t st) {
    dim3 grid((unsigned)((cols + 31) / 32), (unsigned)((ld_dst + 31) / 32)), block(32, 8);
    if (grid.y > 65535) NMG_FAIL(NMG_ERR_UNSUPPORTED, "too many rows for the transpose pre-pass");
    NMG_DISPATCH_DTYPE(dtype, T, (transpose_to_f32_kernel<T><<<grid, block, 0, st>>>(static_cast<const T *>(src), rows, cols, ld_src, dst, ld_dst)));
    NMG_CUDA(cudaGetLastError());
    return NMG_OK;
}

// Same-dtype transpose: src[rows][ld_src] -> dst[cols][ld_dst], 64 x 64 tiles through shared memory.  Both sides move
// 128 bytes (fp32: 256) per warp instruction: a thread reads two neighbouring elements of a source row and writes two
// neighbouring elements of a destination row.  Columns of dst beyond `rows` (up to ld_dst) are zero.
template <typename T>
__global__ void __launch_bounds__(256) transpose_kernel(const T *__restrict__ src, int64_t rows, int64_t cols, int64_t ld_src,
                                                        T *__restrict__ dst, int64_t ld_dst) {
    __shared__ T tile[64][66];
    const int tx = threadIdx.x, ty = threadIdx.y;  // 32 x 8
    const int64_t c0 = (int64_t)blockIdx.x * 64, r0 = (int64_t)blockIdx.y * 64;
    for (int i = ty; i < 64; i += 8) {
        const int64_t r = r0 + i;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int64_t c = c0 + 2 * tx + h;
            tile[i][2 * tx + h] = (r < rows && c < cols) ? src[r * ld_src + c] : DT<T>::from_f32(0.f);
        }
    }
    __syncthreads();
    for (int i = ty; i < 64; i += 8) {
        const int64_t c = c0 + i;
        if (c >= cols) continue;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int64_t r = r0 + 2 * tx + h;
            if (r < ld_dst) dst[c * ld_dst + r] = tile[2 * tx + h][i];
        }
    }
}

int launch_transpose(const void *src, int dtype, int64_t rows, int64_t cols, int64_t ld_src, void *dst, int64_t ld_dst, cudaStream_t st) {
    dim3 block(32, 8);
    const int64_t gy = (ld_dst + 63) / 64;
    if (gy > 65535) NMG_FAIL(NMG_ERR_UNSUPPORTED, "reduction axis too long for the transpose pre-pass");
    dim3 grid((unsigned)((cols + 63) / 64), (unsigned)gy);
    NMG_DISPATCH_DTYPE(dtype, T, (transpose_kernel<T><<<grid, block, 0, st>>>(static_cast<const T *>(src), rows, cols, ld_src, static_cast<T *>(dst), ld_dst)));
    NMG_CUDA(cudaGetLastError());
    return NMG_OK;
}

int launch_widen_to_f32(const void *src, int dtype, int64_t rows, int64_t cols, int64_t ld_src, float *dst,
                        int64_t ld_dst, cudaStream_t st) {
    if (rows > 65535) {
        // fold rows into several launches to stay inside the grid.y limit
        for (int64_t r0 = 0; r0 < rows; r0 += 65535) {
            int64_t nr = rows - r0 < 65535 ? rows - r0 : 65535;
            int rc = launch_widen_to_f32(static_cast<const char *>(src) + r0 * ld_src * dtype_size(dtype), dtype, nr, cols,
                                         ld_src, dst + r0 * ld_dst, ld_dst, st);
            if (rc) return rc;
        }
        return NMG_OK;
    }
    dim3 grid((unsigned)((ld_dst + 255) / 256 > 64 ? 64 : (ld_dst + 255) / 256), (unsigned)rows);
    NMG_DISPATCH_DTYPE(dtype, T, (widen_to_f32_kernel<T><<<grid, 256, 0, st>>>(static_cast<const T *>(src), rows, cols, ld_src, dst, ld_dst)));
    NMG_CUDA(cudaGetLastError());
    return NMG_OK;
}

// ------------------------------------------------------------------------------------------ generic forward kernel
// Any (n, m): one thread per (token, row-block); table driven; reads the caller's activation in place.
struct GenFwdParams {
    const void *val; const int16_t *idx; const void *act; const void *bias; void *out; const int8_t *order;
    int64_t M, K, ntok, ld_act, ld_out, nb, nc;
    int n, m, g, C, cc, token_major, out_token_major;
};
template <typename T>
__global__ void spmm_fwd_generic_kernel(const GenFwdParams prm) {
    const int64_t tok = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t mb = blockIdx.y;
    if (tok >= prm.ntok) return;
    float acc[64];
    for (int r = 0; r < prm.m; r++) acc[r] = 0.f;
    const T *val = static_cast<const T *>(prm.val);
    const T *act = static_cast<const T *>(prm.act);
    for (int64_t kc = 0; kc < prm.nc; kc++) {
        const int64_t tile = kc * prm.nb + mb;
        for (int p = 0; p < prm.C; p++)
            for (int j = 0; j < prm.g; j++) {
                const int slot = p * prm.g + j;
                const int k = prm.idx[tile * prm.cc + slot];
                const int64_t col = kc * prm.cc + k;
                if (k < 0 || k >= prm.cc || col >= prm.K) continue;
                const float x = DT<T>::to_f32(prm.token_major ? act[tok * prm.ld_act + col] : act[col * prm.ld_act + tok]);
                for (int s = 0; s < prm.n; s++)
                    acc[prm.order[p * prm.n + s]] = fmaf(DT<T>::to_f32(val[(tile * prm.cc + slot) * prm.n + s]), x, acc[prm.order[p * prm.n + s]]);
            }
    }
    T *out = static_cast<T *>(prm.out);
    const T *bias = static_cast<const T *>(prm.bias);
    for (int r = 0; r < prm.m; r++) {
        const int64_t row = mb * prm.m + r;
        if (row >= prm.M) break;
        const float o = acc[r] + (bias ? DT<T>::to_f32(bias[row]) : 0.f);
        if (prm.out_token_major) out[tok * prm.ld_out + row] = DT<T>::from_f32(o);
        else out[row * prm.ld_out + tok] = DT<T>::from_f32(o);
    }
}

// ------------------------------------------------------------------------------------------ host side
bool simt_fwd_specialised(int n, int m) {
    return (n == 1 && m == 4) || (n == 2 && m == 4) || (n == 1 && m == 8) || (n == 2 && m == 8) || (n == 1 && m == 16) ||
           (n == 3 && m == 6);
}

// Largest token tile (then two stages before one) whose shared-memory plan fits.
bool choose_fwd(const Geo &geo, size_t es, FwdChoice *c, int *box_rows, int *nbox) {
    const int rbc = kWarps * (16 / geo.m > 0 ? 16 / geo.m : 1);
    *box_rows = geo.cc < 256 ? geo.cc : 256;
    *nbox = (geo.cc + *box_rows - 1) / *box_rows;
    const int tts[3] = {4, 2, 1};
    for (int ti = 0; ti < 3; ti++)
        for (int stages = 2; stages >= 1; stages--) {
            FwdSmemPlan p = fwd_smem_plan(geo.cc, geo.n, rbc, 32 * tts[ti], *nbox, *box_rows, es, stages);
            if (p.total <= 225 * 1024) { c->tt = tts[ti]; c->stages = stages; return true; }
        }
    return false;
}

size_t simt_fwd_workspace_bytes(const Geo &geo, int64_t tokens, int dtype, int layout) {
    if (!simt_fwd_specialised(geo.n, geo.m)) return 0;
    FwdChoice ch; int br, nbx;
    if (!choose_fwd(geo, dtype_size(dtype), &ch, &br, &nbx)) return 0;  // generic kernel, no scratch
    // fp32 activation copy [K][ld], ld padded to the token tile; always taken so the result does not depend
    // on the caller's alignment
    (void)layout;
    return (size_t)geo.K * (size_t)round_up(tokens, 128) * 4 + 256;
}

int simt_fwd(const Geo &geo, int dtype, const void *val, const int16_t *idx, const void *act, int64_t ld_act,
             int64_t tokens, const void *bias, void *out, int64_t ld_out, int layout, void *ws, size_t ws_bytes,
             cudaStream_t st) {
    const bool token_major = layout != NMG_ACT_K_MAJOR;      // activation rows are tokens
    const bool out_token_major = layout == NMG_ACT_TOKEN_MAJOR;
    FwdChoice ch; int box_rows, nbox;
    const bool fast = simt_fwd_specialised(geo.n, geo.m) && choose_fwd(geo, dtype_size(dtype), &ch, &box_rows, &nbox);
    if (!fast) {
        PatternTable tab;
        int rc = get_pattern_table(geo.n, geo.m, &tab);
        if (rc) return rc;
        GenFwdParams p{val, idx, act, bias, out, tab.order, geo.M, geo.K, tokens, ld_act, ld_out, geo.nb, geo.nc,
                       geo.n, geo.m, geo.g, geo.C, geo.cc, token_major ? 1 : 0, out_token_major ? 1 : 0};
        if (geo.nb > 65535) NMG_FAIL(NMG_ERR_UNSUPPORTED, "weight has too many row-blocks for one launch");
        dim3 grid((unsigned)((tokens + 127) / 128), (unsigned)geo.nb);
        const ProfileEvents pe = take_profile_events();
        if (pe.start) NMG_CUDA(cudaEventRecord(pe.start, st));
        NMG_DISPATCH_DTYPE(dtype, T, (spmm_fwd_generic_kernel<T><<<grid, 128, 0, st>>>(p)));
        NMG_CUDA(cudaGetLastError());
        if (pe.stop) NMG_CUDA(cudaEventRecord(pe.stop, st));
        return NMG_OK;
    }
    const size_t need = simt_fwd_workspace_bytes(geo, tokens, dtype, layout);
    if (!ws || ws_bytes < need) NMG_FAIL(NMG_ERR_WORKSPACE, "workspace of %zu bytes required, got %zu", need, ws_bytes);
    float *xt = reinterpret_cast<float *>(((uintptr_t)ws + 255) & ~(uintptr_t)255);
    const int64_t ld_xt = round_up(tokens, 128);
    int rc = token_major ? launch_transpose_to_f32(act, dtype, tokens, geo.K, ld_act, xt, ld_xt, st)
                         : launch_widen_to_f32(act, dtype, geo.K, tokens, ld_act, xt, ld_xt, st);
    if (rc) return rc;

    CUtensorMap tm;
    if ((rc = encode_tmap_2d(&tm, NMG_F32, xt, (uint64_t)ld_xt, (uint64_t)geo.K, (uint64_t)ld_xt, (uint32_t)(32 * ch.tt), (uint32_t)box_rows, 0)))
        return rc;
    int *status = nullptr;
    if ((rc = get_status_word(&status))) return rc;
    const int rbc = kWarps * (16 / geo.m > 0 ? 16 / geo.m : 1);
    FwdParams p{val, idx, bias, out, geo.M, geo.K, tokens, ld_out, geo.nb, geo.nc, geo.g, geo.cc, box_rows, nbox, ch.stages, status};
    const size_t smem = fwd_smem_plan(geo.cc, geo.n, rbc, 32 * ch.tt, nbox, box_rows, dtype_size(dtype), ch.stages).total;

    const ProfileEvents pe = take_profile_events();
    if (pe.start) NMG_CUDA(cudaEventRecord(pe.start, st));
#define NMG_FWD_CASE(N_, M_)                                                                                     \
    if (geo.n == N_ && geo.m == M_) {                                                                            \
        rc = simt_fwd_launch<N_, M_>(dtype, ch.tt, p, tm, rbc, smem, out_token_major, tokens, st);                    \
        if (rc == NMG_OK && pe.stop) NMG_CUDA(cudaEventRecord(pe.stop, st));                                      \
        return rc;                                                                                               \
    }
    NMG_FWD_CASE(1, 4)
    NMG_FWD_CASE(2, 4)
    NMG_FWD_CASE(1, 8)
    NMG_FWD_CASE(2, 8)
    NMG_FWD_CASE(1, 16)
    NMG_FWD_CASE(3, 6)
#undef NMG_FWD_CASE
    NMG_FAIL(NMG_ERR_UNSUPPORTED, "no specialised kernel for %d:%d", geo.n, geo.m);
}

}  // namespace nmg
