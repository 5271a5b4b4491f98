// Shared pieces of the tcgen05 kernels: tile constants, tile order, TMEM / MMA / descriptor primitives and the
// fp32-as-bf16-split tables.  Included by the fused expansion kernel and by the dense-operand kernel.
#pragma once
#include "nmg_common.cuh"

namespace nmg {

constexpr int TC_BM = 128;    // output features per CTA (MMA M)
constexpr int TC_BN = 256;    // tokens per CTA (MMA N)
constexpr int TC_BK = 64;     // reduction elements per stage: one 128-byte swizzle span of 16-bit data
constexpr int TC_STAGES = 4;
constexpr int TC_THREADS = 32 * 14;  // fused kernel: TMA warp, MMA warp, three expansion groups of 4 warps (group 0 also drains)
constexpr int TC_CHUNK_KB = 8;       // fp32 mode: k-blocks (of 64) accumulated in the tensor core before promotion
constexpr int TC_A_BYTES = TC_BM * TC_BK * 2;  // 16 KB
constexpr int TC_B_BYTES = TC_BN * TC_BK * 2;  // 32 KB
constexpr int TC_ACC_COLS = 256;    // one fp32 accumulator tile: 128 lanes x 256 columns

// Tile order: feature tiles are taken in bands of `band_w`; inside a band the CTA index runs over the band's feature
// tiles first, then over token tiles.  The CTAs that are resident together then cover a block of band_w x (CTAs / band_w)
// tiles and share its operand panels through L2; a wave reads band_w weight panels and CTAs / band_w activation
// panels from HBM, which is least when the block is square in bytes: 16 for one-CTA tiles (128 x 256, 148 CTAs), 8 for
// the 256 x 256 tiles of CTA pairs (74 pairs).
constexpr int TC_BAND = 16;
constexpr int TC_BAND_PAIR = 8;
__device__ __forceinline__ void tile_of_cta(int lin, int tiles_f, int tiles_t, int &tf, int &tt, int band_w = TC_BAND) {
    const int per_band = band_w * tiles_t;
    const int band = lin / per_band, within = lin - band * per_band;
    const int width = min(band_w, tiles_f - band * band_w);
    tt = within / width;
    tf = band * band_w + (within - tt * width);
}


__device__ __forceinline__ void tmem_alloc(uint32_t *smem_slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// The same load without the wait, and the wait as a fence on the destination registers: between the two the load is
// in flight and the registers must not be read; the "+r" operands keep the compiler from moving a use above the wait.
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_fence(uint32_t (&r)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
                   "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]),
                   "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]),
                   "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                 :: "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// One 16-byte store to a multicast address: NVSwitch writes it to the same offset on every GPU of the multicast group.
__device__ __forceinline__ void multimem_st_v4(void *mc_addr, uint4 v) {
    asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};"
                 ::"l"(mc_addr), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
                 : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// ---- CTA pairs (thread-block cluster of 2, tcgen05 cta_group::2) -------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local` (a shared::cta address of this CTA) in the CTA with the given cluster rank
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
// Arrive on a barrier of the pair's other CTA (or this one) to say "my reads of the accumulator are done".  The reads are
// tcgen05.ld whose values are already in registers (tcgen05.wait::ld) when this runs, so the signal carries no data and
// needs no release: a release at cluster scope would first wait until every global store this thread has in flight --
// the tile's output -- is acknowledged by L2, once per tile and warp, which is what bounded the drain.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster_bounded(uint64_t *bar, uint32_t parity, int *status, int code) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    for (;;) {
        for (int i = 0; i < 64; i++)
            if (mbar_try_wait_cluster(bar, parity)) return true;
        if (global_timer_ns() - t0 > kWaitLimitNs) break;
    }
    if (status) atomicExch(status, code);
    return false;
}
// 2-D tiled TMA load of a CTA pair, no multicast: the box lands in THIS CTA's shared memory, the bytes are reported to
// the mbarrier at `bar_cluster_addr`, which may live in the peer CTA.
__device__ __forceinline__ void tma_load_2d_pair(void *smem_dst, const CUtensorMap *map, int x, int y, uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(bar_cluster_addr)
        : "memory");
}
// commit of the pair's MMAs: arrives at the barrier at this shared-memory offset in BOTH CTAs
__device__ __forceinline__ void tc2_commit_both(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t *smem_slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc2_mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128 bytes, 8-row groups 1024 bytes
// apart.  Fields: start address >> 4 (bits 0-13), leading byte offset >> 4 (16-29, unused for swizzled K-major,
// set to 1), stride byte offset >> 4 (32-45), descriptor version 1 (46-47), layout type 2 = SWIZZLE_128B (61-63).
__device__ __forceinline__ uint64_t make_sw128_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFF) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
// Instruction descriptor (kind::f16): D = fp32 (bits 4-5 = 1), A / B format (7-9, 10-12: 0 = f16, 1 = bf16), both
// K-major (15, 16 = 0), N >> 3 (17-22), M >> 4 (24-28).
template <typename T> __device__ __forceinline__ uint32_t make_idesc() {
    const uint32_t fmt = sizeof(T) == 2 && DT<T>::id == NMG_BF16 ? 1u : 0u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(TC_BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
}

// Two fp32 values -> two 16-bit values in one word (first in the low half) with one packed conversion.
template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<float>(float, float) { return 0; }  // never used: fp32 outputs are stored as words

template <typename T> __device__ __forceinline__ uint16_t bits16(T v);
template <> __device__ __forceinline__ uint16_t bits16<__half>(__half v) { return __half_as_ushort(v); }
template <> __device__ __forceinline__ uint16_t bits16<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat16_as_ushort(v); }
template <> __device__ __forceinline__ uint16_t bits16<float>(float) { return 0; }  // never used: fp32 outputs are stored as words


// fp32 operands run on the bf16 tensor cores as exact three-way splits x = xh + xm + xl, w = wh + wm + wl.  The
// product keeps the six terms whose weight is >= 2^-16 of the leading one (wh xh, wm xh, wh xm, wm xm, wl xh, wh xl);
// the dropped terms are below 2^-24 relative, the size of an fp32 rounding error.  Each term is one more pass
// over the reduction axis with another pair of planes, accumulated in the same fp32 TMEM tile.
//
// The tensor core's fp32 accumulator truncates instead of rounding, which biases long sums: measured relative error
// grows linearly with the reduction length (3.5e-6 at K = 512, 2.6e-5 at K = 4096).  fp32 mode therefore keeps a
// second accumulator tile in TMEM: every TC_CHUNK_KB k-blocks the first expansion group adds the tensor core's
// partial tile into it with round-to-nearest FADDs (tcgen05.ld / tcgen05.st), and the MMAs restart from zero.  The
// error then no longer depends on K.
template <typename T> struct TcMode { using elem = T; static constexpr int TERMS = 1; static constexpr int GROUPS = 3; };
template <> struct TcMode<float> { using elem = __nv_bfloat16; static constexpr int TERMS = 6; static constexpr int GROUPS = 3; };
static __device__ __constant__ int kSplitW[6] = {0, 1, 0, 1, 2, 0};
static __device__ __constant__ int kSplitX[6] = {0, 0, 1, 1, 0, 2};

}  // namespace nmg
