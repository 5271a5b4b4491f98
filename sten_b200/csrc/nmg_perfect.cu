// Per-block top-n selection without the group constraint ("perfect" n:m): of every m consecutive elements along one
// dimension the n of largest magnitude are kept, in descending order of magnitude, together with their positions.
// Upper bound on the magnitude a grouped n:m layout can keep; the format's quality test compares against it.
//
// The tensor is seen as [outer][size][inner] (size = extent of the sparse dimension, blocks of m along it).  One thread
// owns one (outer, block, inner) triple.  With inner > 1 neighbouring threads read neighbouring addresses (coalesced);
// with inner == 1 a thread's block is contiguous and, for m in {2, 4, 8, 16}, is fetched with 16-byte loads, as are the
// n outputs when they fill whole 16-byte units.  Ties keep the smaller position first.
#include "nmg_common.cuh"

namespace nmg {

struct PerfectParams {
    const void *dense;   // [outer][size][inner]
    void *val;           // [outer][blocks][n][inner]
    int64_t *idx;        // same shape as val
    int64_t outer, size, inner, blocks;
    int n, m;
};

// M_ > 0: block length known at compile time (values live in registers); M_ = 0: any m <= 64, values are re-read.
template <typename T, int M_>
__global__ void __launch_bounds__(256) perfect_select_kernel(PerfectParams p) {
    const int m = M_ > 0 ? M_ : p.m, n = p.n;
    const int64_t total = p.outer * p.blocks * p.inner;
    const T *dense = static_cast<const T *>(p.dense);
    T *val = static_cast<T *>(p.val);
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t in = t % p.inner, bo = t / p.inner, blk = bo % p.blocks, o = bo / p.blocks;
        const T *src = dense + (o * p.size + blk * m) * p.inner + in;
        const int valid = (int)(p.size - blk * m < m ? p.size - blk * m : m);  // positions inside the tensor (the rest is zero padding)
        T *vdst = val + ((o * p.blocks + blk) * n) * p.inner + in;
        int64_t *idst = p.idx + ((o * p.blocks + blk) * n) * p.inner + in;
        uint64_t taken = 0;
        if constexpr (M_ > 0) {
            T v[M_];
            constexpr int V = 16 / (int)sizeof(T);
            if (p.inner == 1 && valid == M_ && (M_ % V) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
#pragma unroll
                for (int u = 0; u < M_ / V; u++) *reinterpret_cast<uint4 *>(&v[u * V]) = __ldg(reinterpret_cast<const uint4 *>(src) + u);
            } else {
#pragma unroll
                for (int r = 0; r < M_; r++) v[r] = r < valid ? src[(int64_t)r * p.inner] : DT<T>::from_f32(0.f);
            }
            for (int j = 0; j < n; j++) {
                float best = -1.f;
                int bi = 0;
#pragma unroll
                for (int r = 0; r < M_; r++) {
                    const float a = fabsf(DT<T>::to_f32(v[r]));
                    if (!((taken >> r) & 1ull) && a > best) { best = a; bi = r; }
                }
                taken |= 1ull << bi;
                T out = DT<T>::from_f32(0.f);
#pragma unroll
                for (int r = 0; r < M_; r++) if (r == bi) out = v[r];
                vdst[(int64_t)j * p.inner] = out;
                idst[(int64_t)j * p.inner] = bi;
            }
        } else {
            for (int j = 0; j < n; j++) {
                float best = -1.f;
                int bi = 0;
                for (int r = 0; r < m; r++) {
                    const float a = r < valid ? fabsf(DT<T>::to_f32(src[(int64_t)r * p.inner])) : 0.f;
                    if (!((taken >> r) & 1ull) && a > best) { best = a; bi = r; }
                }
                taken |= 1ull << bi;
                vdst[(int64_t)j * p.inner] = bi < valid ? src[(int64_t)bi * p.inner] : DT<T>::from_f32(0.f);
                idst[(int64_t)j * p.inner] = bi;
            }
        }
    }
}

// dense[outer][size][inner] from (val, idx); every element of dense is written (zeros included).
template <typename T>
__global__ void __launch_bounds__(256) perfect_densify_kernel(PerfectParams p) {
    const int m = p.m, n = p.n;
    const int64_t total = p.outer * p.blocks * p.inner;
    T *dense = static_cast<T *>(const_cast<void *>(p.dense));
    const T *val = static_cast<const T *>(p.val);
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t in = t % p.inner, bo = t / p.inner, blk = bo % p.blocks, o = bo / p.blocks;
        T *dst = dense + (o * p.size + blk * m) * p.inner + in;
        const int valid = (int)(p.size - blk * m < m ? p.size - blk * m : m);
        const T *vsrc = val + ((o * p.blocks + blk) * n) * p.inner + in;
        const int64_t *isrc = p.idx + ((o * p.blocks + blk) * n) * p.inner + in;
        for (int r = 0; r < valid; r++) {
            T out = DT<T>::from_f32(0.f);
            for (int j = 0; j < n; j++)
                if (isrc[(int64_t)j * p.inner] == r) out = vsrc[(int64_t)j * p.inner];  // later slots win, as a scatter would
            dst[(int64_t)r * p.inner] = out;
        }
    }
}

static int perfect_check(int64_t outer, int64_t size, int64_t inner, int n, int m, int dtype, const void *a, const void *b, const void *c) {
    if (dtype != NMG_F32 && dtype != NMG_F16 && dtype != NMG_BF16) NMG_FAIL(NMG_ERR_INVALID, "dtype must be NMG_F32, NMG_F16 or NMG_BF16, got %d", dtype);
    if (m < 1 || m > 64 || n < 0 || n > m) NMG_FAIL(NMG_ERR_INVALID, "need 0 <= n <= m <= 64, got n=%d m=%d", n, m);
    if (outer < 1 || size < 1 || inner < 1) NMG_FAIL(NMG_ERR_INVALID, "extents must be positive");
    if (!a || !b || !c) NMG_FAIL(NMG_ERR_INVALID, "NULL operand pointer");
    return NMG_OK;
}

}  // namespace nmg

using namespace nmg;

extern "C" int nmg_perfect_nm_select(const void *dense, int64_t outer, int64_t size, int64_t inner, int n, int m, int dtype, void *val,
                                     int64_t *idx, void *stream) {
    int rc = perfect_check(outer, size, inner, n, m, dtype, dense, val, idx);
    if (rc) return rc;
    PerfectParams p{dense, val, idx, outer, size, inner, (size + m - 1) / m, n, m};
    const int64_t total = outer * p.blocks * inner;
    if (n == 0) return NMG_OK;
    const unsigned grid = (unsigned)((total + 255) / 256 < 148 * 64 ? (total + 255) / 256 : 148 * 64);
    cudaStream_t st = (cudaStream_t)stream;
    NMG_DISPATCH_DTYPE(dtype, T, {
        if (m == 2) perfect_select_kernel<T, 2><<<grid, 256, 0, st>>>(p);
        else if (m == 4) perfect_select_kernel<T, 4><<<grid, 256, 0, st>>>(p);
        else if (m == 8) perfect_select_kernel<T, 8><<<grid, 256, 0, st>>>(p);
        else if (m == 16) perfect_select_kernel<T, 16><<<grid, 256, 0, st>>>(p);
        else perfect_select_kernel<T, 0><<<grid, 256, 0, st>>>(p);
    });
    NMG_CUDA(cudaGetLastError());
    return NMG_OK;
}

extern "C" int nmg_perfect_nm_densify(const void *val, const int64_t *idx, int64_t outer, int64_t size, int64_t inner, int n, int m,
                                      int dtype, void *dense, void *stream) {
    int rc = perfect_check(outer, size, inner, n, m, dtype, dense, val, idx);
    if (rc) return rc;
    PerfectParams p{dense, const_cast<void *>(val), const_cast<int64_t *>(idx), outer, size, inner, (size + m - 1) / m, n, m};
    const int64_t total = outer * p.blocks * inner;
    const unsigned grid = (unsigned)((total + 255) / 256 < 148 * 64 ? (total + 255) / 256 : 148 * 64);
    cudaStream_t st = (cudaStream_t)stream;
    NMG_DISPATCH_DTYPE(dtype, T, { perfect_densify_kernel<T><<<grid, 256, 0, st>>>(p); });
    NMG_CUDA(cudaGetLastError());
    return NMG_OK;
}
