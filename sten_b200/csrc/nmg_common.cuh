// Shared declarations of the nmg_b200 library: error reporting, dtype helpers, compile-time pattern tables,
// per-device resources (pattern tables, status word), and the bounded mbarrier / TMA primitives.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/nmg_b200.h"

namespace nmg {

// ------------------------------------------------------------------------------------------------ errors
void set_error(const char *fmt, ...);
#define NMG_FAIL(code, ...)          \
    do {                             \
        ::nmg::set_error(__VA_ARGS__); \
        return (code);               \
    } while (0)
#define NMG_CUDA(call)                                                                              \
    do {                                                                                            \
        cudaError_t e__ = (call);                                                                   \
        if (e__ != cudaSuccess) NMG_FAIL(NMG_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(e__)); \
    } while (0)

// ------------------------------------------------------------------------------------------------ geometry
struct Geo {
    int n, m, g;
    int C;        // patterns per chunk = comb(m, n)
    int cc;       // columns per chunk = C * g
    int64_t M, K; // logical weight shape
    int64_t nb;   // row-blocks   = ceil(M / m)
    int64_t nc;   // column chunks = ceil(K / cc)
};
int make_geo(int64_t M, int64_t K, int n, int m, int g, Geo *out); // validates, sets last error

// ------------------------------------------------------------------------------------------------ pattern order
// Revolving-door list of the n-subsets of [0, m): neighbours differ in one element.  Same recursion as the
// format definition (first the subsets without m-1, reversed when `flip`, then those with it); constexpr so
// that kernels specialised on (n, m) see the table as immediates.
constexpr int64_t comb(int n, int m) {
    if (n < 0 || n > m) return 0;
    int64_t r = 1;
    for (int i = 1; i <= n; i++) r = r * (m - n + i) / i;
    return r;
}
constexpr int gen_order(int n, int m, bool flip, int8_t *out, int ld) {
    if (n == m || n == 0) {
        for (int i = 0; i < n; i++) out[i] = (int8_t)i;
        return 1;
    }
    int c1 = gen_order(n, m - 1, true, out, ld);
    if (flip) {
        for (int a = 0, b = c1 - 1; a < b; a++, b--)
            for (int i = 0; i < n; i++) {
                int8_t t = out[a * ld + i];
                out[a * ld + i] = out[b * ld + i];
                out[b * ld + i] = t;
            }
    }
    int c2 = gen_order(n - 1, m - 1, !flip, out + c1 * ld, ld);
    for (int r = 0; r < c2; r++) out[(c1 + r) * ld + (n - 1)] = (int8_t)(m - 1);
    return c1 + c2;
}
template <int N_, int M_>
struct Order {
    static constexpr int C = (int)comb(N_, M_);
    static constexpr int LD = N_ > 0 ? N_ : 1;
    int8_t v[C * LD];  // flat so that the generator's pointer arithmetic stays inside one array
    constexpr Order() : v{} { gen_order(N_, M_, false, v, LD); }
    constexpr int row(int p, int s) const { return v[p * LD + s]; }
};

// Device copy of order[C][n] followed by slot_of_row[C][m] (position of row r inside pattern p, or -1),
// created once per (device, n, m) and never freed.
struct PatternTable {
    const int8_t *order;       // [C][n]
    const int8_t *slot_of_row; // [C][m]
};
int get_pattern_table(int n, int m, PatternTable *out);

// Events requested through nmg_profile_next for the calling thread; take_profile_events hands them out once.
struct ProfileEvents { cudaEvent_t start, stop; };
ProfileEvents take_profile_events();

// One int per device that kernels set to a non-zero code when a bounded wait runs out.
// the weight-expansion pass of the matmul path used as the densifier (nmg_gemm_tc.cu)
bool tc_expand_plain_supported(const Geo &geo, int dtype, const void *dense, int64_t ld);
int tc_expand_plain(const Geo &geo, int dtype, const void *val, const int16_t *idx, void *dense, int64_t ld, cudaStream_t st);
int get_status_word(int **dev_ptr);
int get_wave_counter(unsigned **dev_ptr);  // one of a few rotating 4-byte counters of the current device (spare bytes of the status block)
// Status word of nmg_spmm_noalloc on device `dev` (start of the built-in scratch array), or NULL before its first call there.
int *noalloc_status_word(int dev);

// ------------------------------------------------------------------------------------------------ dtypes
template <typename T> struct DT;
template <> struct DT<float> {
    static constexpr int id = NMG_F32;
    __device__ static __forceinline__ float to_f32(float v) { return v; }
    __device__ static __forceinline__ float from_f32(float v) { return v; }
};
template <> struct DT<__half> {
    static constexpr int id = NMG_F16;
    __device__ static __forceinline__ float to_f32(__half v) { return __half2float(v); }
    __device__ static __forceinline__ __half from_f32(float v) { return __float2half_rn(v); }
};
template <> struct DT<__nv_bfloat16> {
    static constexpr int id = NMG_BF16;
    __device__ static __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ static __forceinline__ __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }
};
inline size_t dtype_size(int dtype) { return dtype == NMG_F32 ? 4 : 2; }

#define NMG_DISPATCH_DTYPE(dtype, T, ...)                                   \
    do {                                                                    \
        if ((dtype) == NMG_F32) { using T = float; __VA_ARGS__; }           \
        else if ((dtype) == NMG_F16) { using T = __half; __VA_ARGS__; }     \
        else { using T = __nv_bfloat16; __VA_ARGS__; }                      \
    } while (0)

// ------------------------------------------------------------------------------------------------ device primitives
#ifdef __CUDACC__
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after about two seconds of wall-clock time (%globaltimer, checked every 64 polls; each poll
// may itself sleep for a hardware-defined slice), records `code` in the status word and reports failure so the caller
// can leave the kernel.  Two seconds is far above any healthy wait of these kernels and keeps a lost hand-off from
// occupying the GPU.
constexpr uint64_t kWaitLimitNs = 2000000000ull;
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Soft rendezvous of the persistent CTAs of one launch: count this CTA in and wait until `target` CTAs have been counted
// or `limit_ns` have passed, whichever comes first.  It only keeps CTAs that share operand panels through L2 in step;
// nothing depends on it having been reached, so a CTA that is late or absent costs the others at most the limit.
__device__ __forceinline__ void soft_rendezvous(unsigned *ctr, unsigned target, uint64_t limit_ns) {
    atomicAdd(ctr, 1u);
    const uint64_t t0 = global_timer_ns();
    while (*reinterpret_cast<volatile unsigned *>(ctr) < target) {
        if (global_timer_ns() - t0 > limit_ns) break;
        __nanosleep(40);
    }
}
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, int *status, int code,
                                                  uint64_t limit_ns = kWaitLimitNs) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    for (;;) {
        for (int i = 0; i < 64; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (global_timer_ns() - t0 > limit_ns) break;
    }
    if (status) atomicExch(status, code);
    return false;
}
// 2-D tiled TMA load, no multicast: box at (x = inner coordinate, y = outer coordinate) -> shared memory.
__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
// Tiled store shared -> global of one box (bulk async-group completion).  Rows and columns of the box that fall outside
// the tensor are not written.  x * element size must be a multiple of 16 bytes and neither coordinate may be negative.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, const void *smem_src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// all bulk stores of this thread have finished READING shared memory: the source may be overwritten or given up
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void cp_async_16(void *smem_dst, const void *gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Queue an asynchronous copy of the byte range [src, src + bytes) into shared memory with 16-byte cp.async.
// The range is widened to 16-byte boundaries; `dst16` must be 16-byte aligned and hold bytes + 32.  Returns
// where the first requested byte lands.  The widened bytes lie in the 16-byte blocks that already contain
// requested data, so they are inside the same allocation granule.
__device__ __forceinline__ const char *stage_bytes_async(char *dst16, const void *src, int64_t bytes, int tid, int nthr) {
    uintptr_t s = (uintptr_t)src;
    uintptr_t s0 = s & ~(uintptr_t)15;
    int head = (int)(s - s0);
    int64_t blocks = (head + bytes + 15) >> 4;
    for (int64_t b = tid; b < blocks; b += nthr) cp_async_16(dst16 + (b << 4), (const char *)s0 + (b << 4));
    return dst16 + head;
}
#endif  // __CUDACC__

// Host: encode a 2-D tiled tensor map (row-major [rows][ld] array, box = box_rows x box_cols) without linking libcuda.
int encode_tmap_2d(CUtensorMap *map, int dtype, const void *base, uint64_t cols, uint64_t rows, uint64_t ld_elems,
                   uint32_t box_cols, uint32_t box_rows, int swizzle_128b);

}  // namespace nmg
