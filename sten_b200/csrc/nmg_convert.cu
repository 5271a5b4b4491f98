// Format conversion kernels: dense -> nmg magnitude sparsifier (bit-exact with the sequential definition of the
// format) and nmg -> dense.  Both are one pass over the weight; the weight is read / written in place in its
// [batch][M][K] layout, so no padded, permuted or zero-filled temporaries exist.
#include "nmg_common.cuh"

namespace nmg {

// =====================================================================================================
// Sparsifier.
//
// Definition of the result (the reference's CPU implementation): for every tile, score each (column c, pattern p)
// with the fp32 sum of |w| over the rows of p (summed in slot order), sort all (score, c, p) triples
// descending (ties: larger c, then larger p) and walk the list once, accepting a triple when its column is
// still free and its pattern holds fewer than g columns.
//
// Equivalent selection used here (one warp per tile): every free column remembers its best pattern among
// the patterns that still have room; each round the warp takes the maximum (score, c, p) over the free
// columns with two warp reductions, appends c to pattern p, and only when p becomes full do the columns that
// pointed at p re-evaluate.  The sequence of accepted triples is identical to the sorted walk, so val / idx
// are identical bit for bit, without the C^2*g-element sort and without scratch memory in HBM.
// =====================================================================================================

struct SparsifyParams {
    const void *dense;
    void *val;
    int16_t *idx;
    const int8_t *order;  // [C][n] device
    int64_t M, K, ld, batch_stride;
    int64_t nb, nc, tiles;
    int n, m, g, C, cc;
    int slab_bytes;  // shared memory per warp
};

__device__ __forceinline__ void eval_column(const float *x, const int8_t *ord, const int16_t *cnt, int c, int cc, int n,
                                            int g, int C, uint32_t &best_s, int &best_p) {
    best_s = 0;
    best_p = -1;
    for (int p = 0; p < C; p++) {
        if (cnt[p] >= g) continue;
        float s = 0.f;
        for (int i = 0; i < n; i++) s = __fadd_rn(s, fabsf(x[(int)ord[p * n + i] * cc + c]));
        uint32_t b = __float_as_uint(s);
        if (best_p < 0 || b >= best_s) {  // ties go to the larger pattern index
            best_s = b;
            best_p = p;
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256) sparsify_kernel(SparsifyParams prm) {
    extern __shared__ __align__(16) char smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int n = prm.n, m = prm.m, g = prm.g, C = prm.C, cc = prm.cc;

    // CTA-wide copy of the pattern table, then one slab per warp.
    int8_t *ord = reinterpret_cast<int8_t *>(smem);
    const int ord_bytes = (C * n + 15) & ~15;
    for (int i = threadIdx.x; i < C * n; i += blockDim.x) ord[i] = prm.order[i];
    __syncthreads();

    char *slab = smem + ord_bytes + (size_t)warp * prm.slab_bytes;
    float *x = reinterpret_cast<float *>(slab);                         // [m][cc]
    uint32_t *col_score = reinterpret_cast<uint32_t *>(x + (size_t)m * cc);  // [cc]
    int16_t *col_pat = reinterpret_cast<int16_t *>(col_score + cc);      // [cc], -1 = column taken
    int16_t *out_idx = col_pat + cc;                                     // [cc]
    int16_t *cnt = out_idx + cc;                                         // [C]

    const T *dense = static_cast<const T *>(prm.dense);
    T *val = static_cast<T *>(prm.val);

    for (int64_t tile = (int64_t)blockIdx.x * nwarps + warp; tile < prm.tiles; tile += (int64_t)gridDim.x * nwarps) {
        const int64_t mb = tile % prm.nb, kc = (tile / prm.nb) % prm.nc, b = tile / (prm.nb * prm.nc);
        const int64_t row0 = mb * m, col0 = kc * cc;
        const T *src = dense + b * prm.batch_stride;
        for (int r = 0; r < m; r++) {
            const bool row_ok = row0 + r < prm.M;
            const T *srow = src + (row0 + r) * prm.ld + col0;
            for (int c = lane; c < cc; c += 32)
                x[r * cc + c] = (row_ok && col0 + c < prm.K) ? DT<T>::to_f32(srow[c]) : 0.f;
        }
        for (int p = lane; p < C; p += 32) cnt[p] = 0;
        __syncwarp();

        uint32_t my_s = 0, my_cp = 0;  // best free column of this lane; my_cp = ((c << 16) | p) + 1, 0 = none
        for (int c = lane; c < cc; c += 32) {
            uint32_t s; int p;
            eval_column(x, ord, cnt, c, cc, n, g, C, s, p);
            col_score[c] = s;
            col_pat[c] = (int16_t)p;
            uint32_t cp = (((uint32_t)c << 16) | (uint32_t)p) + 1;
            if (s > my_s || (s == my_s && cp > my_cp)) { my_s = s; my_cp = cp; }
        }
        __syncwarp();

        for (int round = 0; round < cc; round++) {
            const uint32_t top_s = __reduce_max_sync(0xffffffffu, my_cp ? my_s : 0u);
            const uint32_t top_cp = __reduce_max_sync(0xffffffffu, (my_cp && my_s == top_s) ? my_cp : 0u);
            if (top_cp == 0) break;  // cannot happen for a well-formed tile; keeps the loop bounded anyway
            const int c = (int)((top_cp - 1) >> 16), p = (int)((top_cp - 1) & 0xffffu);
            const int j = cnt[p];
            const bool owner = (c & 31) == lane;
            __syncwarp();
            if (lane == 0) { out_idx[p * g + j] = (int16_t)c; cnt[p] = (int16_t)(j + 1); }
            if (owner) col_pat[c] = -1;
            __syncwarp();
            const bool filled = (j + 1 == g);
            if (filled) {
                for (int c2 = lane; c2 < cc; c2 += 32)
                    if (col_pat[c2] == p) {
                        uint32_t s; int p2;
                        eval_column(x, ord, cnt, c2, cc, n, g, C, s, p2);
                        col_score[c2] = s;
                        col_pat[c2] = (int16_t)p2;
                    }
            }
            if (filled || owner) {
                my_s = 0; my_cp = 0;
                for (int c2 = lane; c2 < cc; c2 += 32) {
                    const int p2 = col_pat[c2];
                    if (p2 < 0) continue;
                    const uint32_t s = col_score[c2];
                    const uint32_t cp = (((uint32_t)c2 << 16) | (uint32_t)p2) + 1;
                    if (my_cp == 0 || s > my_s || (s == my_s && cp > my_cp)) { my_s = s; my_cp = cp; }
                }
            }
        }
        __syncwarp();

        int16_t *idx_out = prm.idx + tile * cc;
        T *val_out = val + tile * (int64_t)cc * n;
        for (int s = lane; s < cc; s += 32) idx_out[s] = out_idx[s];
        for (int e = lane; e < cc * n; e += 32) {
            const int s = e / n, t = e - s * n;
            const int c = out_idx[s], p = s / g;
            val_out[e] = DT<T>::from_f32(x[(int)ord[p * n + t] * cc + c]);
        }
        __syncwarp();
    }
}

// =====================================================================================================
// Densifier: one CTA per tile.  The tile's idx is inverted in shared memory (column -> slot), val is staged,
// and the m x cc block is written row by row with coalesced stores; zeros are produced by the same stores, so
// the output needs no separate clearing pass.
// =====================================================================================================
struct DensifyParams {
    const void *val;
    const int16_t *idx;
    void *dense;
    const int8_t *slot_of_row;  // [C][m] device
    int64_t M, K, ld, batch_stride;
    int64_t nb, nc, tiles;
    int n, m, g, C, cc;
};

template <typename T>
__global__ void __launch_bounds__(128) densify_kernel(DensifyParams prm) {
    extern __shared__ __align__(16) char smem[];
    const int n = prm.n, m = prm.m, g = prm.g, C = prm.C, cc = prm.cc;
    T *sval = reinterpret_cast<T *>(smem);                                             // [cc][n]
    int16_t *pos = reinterpret_cast<int16_t *>(smem + (((size_t)cc * n * sizeof(T) + 15) & ~(size_t)15));  // [cc]
    int8_t *sor = reinterpret_cast<int8_t *>(pos + cc);                                // [C][m]
    for (int i = threadIdx.x; i < C * m; i += blockDim.x) sor[i] = prm.slot_of_row[i];

    const T *val = static_cast<const T *>(prm.val);
    T *dense = static_cast<T *>(prm.dense);
    for (int64_t tile = blockIdx.x; tile < prm.tiles; tile += gridDim.x) {
        const int64_t mb = tile % prm.nb, kc = (tile / prm.nb) % prm.nc, b = tile / (prm.nb * prm.nc);
        __syncthreads();
        for (int c = threadIdx.x; c < cc; c += blockDim.x) pos[c] = -1;
        const T *vsrc = val + tile * (int64_t)cc * n;
        for (int e = threadIdx.x; e < cc * n; e += blockDim.x) sval[e] = vsrc[e];
        __syncthreads();
        const int16_t *isrc = prm.idx + tile * cc;
        for (int s = threadIdx.x; s < cc; s += blockDim.x) {
            const int c = isrc[s];
            if (c >= 0 && c < cc) pos[c] = (int16_t)s;  // a malformed index is ignored, never dereferenced
        }
        __syncthreads();
        T *dst = dense + b * prm.batch_stride;
        for (int r = 0; r < m; r++) {
            const int64_t row = mb * m + r;
            if (row >= prm.M) break;
            T *drow = dst + row * prm.ld + kc * cc;
            for (int c = threadIdx.x; c < cc; c += blockDim.x) {
                if (kc * cc + c >= prm.K) break;
                const int s = pos[c];
                T v = DT<T>::from_f32(0.f);
                if (s >= 0) {
                    const int t = sor[(s / g) * m + r];
                    if (t >= 0) v = sval[s * n + t];
                }
                drow[c] = v;
            }
        }
    }
}

static int sm_count() {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return sms > 0 ? sms : 148;
}

static int check_dtype(int dtype) {
    if (dtype != NMG_F32 && dtype != NMG_F16 && dtype != NMG_BF16)
        NMG_FAIL(NMG_ERR_INVALID, "dtype must be NMG_F32, NMG_F16 or NMG_BF16, got %d", dtype);
    return NMG_OK;
}

}  // namespace nmg

using namespace nmg;

extern "C" int nmg_sparsify(const void *dense, int64_t batch, int64_t M, int64_t K, int64_t ld_dense,
                            int64_t batch_stride, int n, int m, int g, int dtype, void *val, int16_t *idx,
                            void *stream) {
    Geo geo;
    int rc = make_geo(M, K, n, m, g, &geo);
    if (rc) return rc;
    if ((rc = check_dtype(dtype))) return rc;
    if (!dense || !val || !idx) NMG_FAIL(NMG_ERR_INVALID, "dense, val and idx must be non-NULL");
    if (n < 1) NMG_FAIL(NMG_ERR_INVALID, "the sparsifier needs n >= 1");
    if (batch < 1 || ld_dense < K || (batch > 1 && batch_stride < M * ld_dense))
        NMG_FAIL(NMG_ERR_INVALID, "bad batch / leading dimension (batch=%lld ld=%lld)", (long long)batch, (long long)ld_dense);
    PatternTable tab;
    if ((rc = get_pattern_table(n, m, &tab))) return rc;

    SparsifyParams p{};
    p.dense = dense; p.val = val; p.idx = idx; p.order = tab.order;
    p.M = M; p.K = K; p.ld = ld_dense; p.batch_stride = batch_stride;
    p.nb = geo.nb; p.nc = geo.nc; p.tiles = batch * geo.nb * geo.nc;
    p.n = n; p.m = m; p.g = g; p.C = geo.C; p.cc = geo.cc;
    size_t slab = (size_t)m * geo.cc * 4 + (size_t)geo.cc * 4 + (size_t)geo.cc * 2 * 2 + (size_t)geo.C * 2;
    slab = (slab + 15) & ~(size_t)15;
    const size_t ord_bytes = ((size_t)geo.C * n + 15) & ~(size_t)15;
    const size_t budget = 200 * 1024;
    if (ord_bytes + slab > budget)
        NMG_FAIL(NMG_ERR_UNSUPPORTED, "tile of m=%d x %d columns needs %zu bytes of shared memory (limit %zu)", m, geo.cc,
                 ord_bytes + slab, budget);
    int warps = (int)((budget - ord_bytes) / slab);
    if (warps > 8) warps = 8;
    // keep several CTAs per SM resident when the slab is small
    while (warps > 2 && (ord_bytes + warps * slab) > 56 * 1024) warps--;
    p.slab_bytes = (int)slab;
    const size_t smem = ord_bytes + warps * slab;
    int64_t ctas = (p.tiles + warps - 1) / warps;
    const int64_t max_ctas = (int64_t)sm_count() * 16;
    if (ctas > max_ctas) ctas = max_ctas;
    cudaStream_t st = (cudaStream_t)stream;
    NMG_DISPATCH_DTYPE(dtype, T, {
        NMG_CUDA(cudaFuncSetAttribute(sparsify_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        sparsify_kernel<T><<<(unsigned)ctas, warps * 32, smem, st>>>(p);
    });
    NMG_CUDA(cudaGetLastError());
    return NMG_OK;
}

extern "C" int nmg_densify(const void *val, const int16_t *idx, int64_t batch, int64_t M, int64_t K, int n, int m,
                           int g, int dtype, void *dense, int64_t ld_dense, int64_t batch_stride, void *stream) {
    Geo geo;
    int rc = make_geo(M, K, n, m, g, &geo);
    if (rc) return rc;
    if ((rc = check_dtype(dtype))) return rc;
    if (!dense || !val || !idx) NMG_FAIL(NMG_ERR_INVALID, "dense, val and idx must be non-NULL");
    if (batch < 1 || ld_dense < K || (batch > 1 && batch_stride < M * ld_dense))
        NMG_FAIL(NMG_ERR_INVALID, "bad batch / leading dimension (batch=%lld ld=%lld)", (long long)batch, (long long)ld_dense);
    PatternTable tab;
    if ((rc = get_pattern_table(n, m, &tab))) return rc;

    DensifyParams p{};
    p.val = val; p.idx = idx; p.dense = dense; p.slot_of_row = tab.slot_of_row;
    p.M = M; p.K = K; p.ld = ld_dense; p.batch_stride = batch_stride;
    p.nb = geo.nb; p.nc = geo.nc; p.tiles = batch * geo.nb * geo.nc;
    p.n = n; p.m = m; p.g = g; p.C = geo.C; p.cc = geo.cc;
    const size_t es = dtype_size(dtype);
    const size_t smem = (((size_t)geo.cc * n * es + 15) & ~(size_t)15) + (size_t)geo.cc * 2 + (size_t)geo.C * m;
    if (smem > 200 * 1024)
        NMG_FAIL(NMG_ERR_UNSUPPORTED, "tile of %d columns needs %zu bytes of shared memory (limit %d)", geo.cc, smem, 200 * 1024);
    int64_t ctas = p.tiles;
    const int64_t max_ctas = (int64_t)sm_count() * 32;
    if (ctas > max_ctas) ctas = max_ctas;
    cudaStream_t st = (cudaStream_t)stream;
    NMG_DISPATCH_DTYPE(dtype, T, {
        NMG_CUDA(cudaFuncSetAttribute(densify_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        densify_kernel<T><<<(unsigned)ctas, 128, smem, st>>>(p);
    });
    NMG_CUDA(cudaGetLastError());
    return NMG_OK;
}
