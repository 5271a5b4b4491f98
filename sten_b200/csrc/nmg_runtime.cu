// Host-side runtime of the nmg_b200 library: thread-local error text, argument validation, per-device
// pattern tables and status word, tensor-map encoding.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <atomic>
#include <mutex>
#include <tuple>
#include <vector>

#include "nmg_common.cuh"

namespace nmg {

static thread_local char g_err[512] = "";

void set_profile_events(cudaEvent_t a, cudaEvent_t b);

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int make_geo(int64_t M, int64_t K, int n, int m, int g, Geo *out) {
    if (m < 1 || m > 64 || n < 0 || n > m) NMG_FAIL(NMG_ERR_INVALID, "need 0 <= n <= m <= 64, got n=%d m=%d", n, m);
    if (g < 1) NMG_FAIL(NMG_ERR_INVALID, "group size must be >= 1, got %d", g);
    if (M < 1 || K < 1) NMG_FAIL(NMG_ERR_INVALID, "weight shape must be positive, got %lld x %lld", (long long)M, (long long)K);
    int64_t C = comb(n, m);
    if (C * g >= 32768) NMG_FAIL(NMG_ERR_INVALID, "comb(m,n)*g = %lld does not fit the int16 index (must be < 32768)", (long long)(C * g));
    out->n = n; out->m = m; out->g = g;
    out->C = (int)C; out->cc = (int)(C * g);
    out->M = M; out->K = K;
    out->nb = (M + m - 1) / m;
    out->nc = (K + out->cc - 1) / out->cc;
    return NMG_OK;
}

static thread_local ProfileEvents g_prof = {nullptr, nullptr};
ProfileEvents take_profile_events() {
    ProfileEvents e = g_prof;
    g_prof = {nullptr, nullptr};
    return e;
}
void set_profile_events(cudaEvent_t a, cudaEvent_t b) { g_prof = {a, b}; }

// ------------------------------------------------------------------------------------------------ per-device caches
static std::mutex g_mu;
static std::map<std::tuple<int, int, int>, PatternTable> g_tables;
static std::map<int, int *> g_status;

int get_pattern_table(int n, int m, PatternTable *out) {
    int dev = 0;
    NMG_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(g_mu);
    auto key = std::make_tuple(dev, n, m);
    auto it = g_tables.find(key);
    if (it != g_tables.end()) { *out = it->second; return NMG_OK; }
    int C = (int)comb(n, m);
    int nn = n > 0 ? n : 1;
    std::vector<int8_t> host((size_t)C * nn + (size_t)C * m, (int8_t)-1);
    gen_order(n, m, false, host.data(), nn);
    int8_t *sor = host.data() + (size_t)C * nn;
    for (int p = 0; p < C; p++)
        for (int s = 0; s < n; s++) sor[p * m + host[p * nn + s]] = (int8_t)s;
    int8_t *dev_buf = nullptr;
    NMG_CUDA(cudaMalloc(&dev_buf, host.size()));
    NMG_CUDA(cudaMemcpy(dev_buf, host.data(), host.size(), cudaMemcpyHostToDevice));
    PatternTable t{dev_buf, dev_buf + (size_t)C * nn};
    g_tables[key] = t;
    *out = t;
    return NMG_OK;
}

int get_status_word(int **dev_ptr) {
    int dev = 0;
    NMG_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_status.find(dev);
    if (it == g_status.end()) {
        int *p = nullptr;
        NMG_CUDA(cudaMalloc(&p, 256));
        NMG_CUDA(cudaMemset(p, 0, 256));
        it = g_status.emplace(dev, p).first;
    }
    *dev_ptr = it->second;
    return NMG_OK;
}

// Bytes 64..191 of the status block: 32 counters handed out in rotation, so that launches in flight on different streams
// use different ones.  The caller zeroes its counter on its stream before the launch that uses it.
int get_wave_counter(unsigned **dev_ptr) {
    static std::atomic<unsigned> next{0};
    int *status = nullptr;
    int rc = get_status_word(&status);
    if (rc) return rc;
    *dev_ptr = reinterpret_cast<unsigned *>(status) + 16 + (next.fetch_add(1) % 32);
    return NMG_OK;
}

// The status word of the current device if one exists already, else NULL; never allocates.
static int *peek_status_word(int dev) {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_status.find(dev);
    return it == g_status.end() ? nullptr : it->second;
}

// ------------------------------------------------------------------------------------------------ tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

int encode_tmap_2d(CUtensorMap *map, int dtype, const void *base, uint64_t cols, uint64_t rows, uint64_t ld_elems,
                   uint32_t box_cols, uint32_t box_rows, int swizzle_128b) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) NMG_FAIL(NMG_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    size_t es = dtype_size(dtype);
    if (((uintptr_t)base & 15) || ((ld_elems * es) & 15))
        NMG_FAIL(NMG_ERR_INVALID, "TMA operand needs a 16-byte aligned base and row pitch");
    CUtensorMapDataType dt = dtype == NMG_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                             : dtype == NMG_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld_elems * es};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, dt, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle_128b ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) NMG_FAIL(NMG_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return NMG_OK;
}

}  // namespace nmg

// ------------------------------------------------------------------------------------------------ C ABI (host-only part)
extern "C" {

int nmg_version(void) { return 100; }

const char *nmg_last_error(void) { return nmg::g_err; }

int64_t nmg_num_patterns(int n, int m) { return nmg::comb(n, m); }

int nmg_pattern_order(int n, int m, int8_t *order_out) {
    if (!order_out) NMG_FAIL(NMG_ERR_INVALID, "order_out is NULL");
    if (m < 1 || m > 64 || n < 0 || n > m) NMG_FAIL(NMG_ERR_INVALID, "need 0 <= n <= m <= 64");
    nmg::gen_order(n, m, false, order_out, n > 0 ? n : 1);
    return NMG_OK;
}

int nmg_profile_next(void *start_event, void *stop_event) {
    if (!start_event || !stop_event) NMG_FAIL(NMG_ERR_INVALID, "both events must be non-NULL");
    nmg::set_profile_events((cudaEvent_t)start_event, (cudaEvent_t)stop_event);
    return NMG_OK;
}

int nmg_memcpy_2d_async(void *dst, size_t dst_pitch, const void *src, size_t src_pitch, size_t width_bytes, size_t rows,
                        void *stream) {
    if (!dst || !src) NMG_FAIL(NMG_ERR_INVALID, "NULL pointer");
    if (width_bytes == 0 || rows == 0) return NMG_OK;
    if (dst_pitch < width_bytes || src_pitch < width_bytes) NMG_FAIL(NMG_ERR_INVALID, "pitch smaller than the row width");
    NMG_CUDA(cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, rows, cudaMemcpyDefault, (cudaStream_t)stream));
    return NMG_OK;
}

// Two words can exist per device: the allocated one every workspace-taking entry point hands to its kernels, and the
// first word of the built-in scratch array that nmg_spmm_noalloc uses.  Both are read (whichever exist); nothing is
// allocated here, so a caller that only ever uses nmg_spmm_noalloc can still ask for the status.
int nmg_read_status(void *stream, int *status_out) {
    if (!status_out) NMG_FAIL(NMG_ERR_INVALID, "status_out is NULL");
    int dev = 0;
    NMG_CUDA(cudaGetDevice(&dev));
    int *words[2] = {nmg::peek_status_word(dev), nmg::noalloc_status_word(dev)};
    int codes[2] = {0, 0};
    cudaStream_t st = (cudaStream_t)stream;
    for (int i = 0; i < 2; i++)
        if (words[i]) NMG_CUDA(cudaMemcpyAsync(&codes[i], words[i], sizeof(int), cudaMemcpyDeviceToHost, st));
    NMG_CUDA(cudaStreamSynchronize(st));
    *status_out = codes[0] ? codes[0] : codes[1];
    if (*status_out != 0) {
        for (int i = 0; i < 2; i++)
            if (words[i] && codes[i]) NMG_CUDA(cudaMemsetAsync(words[i], 0, sizeof(int), st));
        NMG_FAIL(NMG_ERR_TIMEOUT, "a device-side bounded wait ran out (code %d)", *status_out);
    }
    return NMG_OK;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------ wait self-test
namespace nmg {
// One thread waits, with the library's bounded wait, on an mbarrier that nothing ever arrives at.  The wait gives up after
// `limit_ns`, records code 90 in the status word and the kernel returns normally.
__global__ void selftest_wait_kernel(int *status, unsigned long long limit_ns) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
        mbar_wait_bounded(&bar, 0, status, 90, limit_ns);
    }
}
}  // namespace nmg

extern "C" int nmg_selftest_wait(uint64_t limit_ns, void *stream) {
    if (limit_ns == 0 || limit_ns > 1000000000ull) NMG_FAIL(NMG_ERR_INVALID, "limit_ns must be between 1 and 1e9 (one second)");
    int *status = nullptr;
    int rc = nmg::get_status_word(&status);
    if (rc) return rc;
    nmg::selftest_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status, (unsigned long long)limit_ns);
    NMG_CUDA(cudaGetLastError());
    return NMG_OK;
}

// ------------------------------------------------------------------------------------------------ fp32 FMA peak
namespace nmg {
__global__ void __launch_bounds__(256) fma_peak_kernel(float *sink, int iters, float a, float b) {
    float r[16];
#pragma unroll
    for (int i = 0; i < 16; i++) r[i] = (float)(threadIdx.x + i);
    for (int it = 0; it < iters; it++) {
#pragma unroll
        for (int u = 0; u < 4; u++)
#pragma unroll
            for (int i = 0; i < 16; i++) r[i] = fmaf(r[i], a, b);
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 16; i++) s += r[i];
    if (s == 123.456f) sink[0] = s;  // keeps the loop alive without a store on the timed path
}
}  // namespace nmg

extern "C" int nmg_measure_fma_peak(double *tflops_out, void *stream) {
    if (!tflops_out) NMG_FAIL(NMG_ERR_INVALID, "tflops_out is NULL");
    cudaStream_t st = (cudaStream_t)stream;
    int dev = 0, sms = 0;
    NMG_CUDA(cudaGetDevice(&dev));
    NMG_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    int *status = nullptr;
    int rc = nmg::get_status_word(&status);
    if (rc) return rc;
    float *sink = reinterpret_cast<float *>(status) + 8;  // spare bytes of the 256-byte status block
    const int iters = 4096, blocks = sms * 8, threads = 256;
    cudaEvent_t e0, e1;
    NMG_CUDA(cudaEventCreate(&e0));
    NMG_CUDA(cudaEventCreate(&e1));
    double best = 0.0;
    for (int rep = 0; rep < 6; rep++) {
        NMG_CUDA(cudaEventRecord(e0, st));
        nmg::fma_peak_kernel<<<blocks, threads, 0, st>>>(sink, iters, 0.999f, 0.001f);
        NMG_CUDA(cudaEventRecord(e1, st));
        NMG_CUDA(cudaEventSynchronize(e1));
        float ms = 0.f;
        NMG_CUDA(cudaEventElapsedTime(&ms, e0, e1));
        const double flops = 2.0 * 64.0 * iters * (double)blocks * threads;
        if (rep >= 2 && ms > 0.f && flops / (ms * 1e-3) / 1e12 > best) best = flops / (ms * 1e-3) / 1e12;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    NMG_CUDA(cudaGetLastError());
    *tflops_out = best;
    return NMG_OK;
}
