// Shared device/host helpers for the sm_100a sparse-KV decode kernels.
//
// Everything here is header-only: PTX wrappers for mbarrier, TMA
// (cp.async.bulk.tensor), ldmatrix and mma.sync, warp reductions, and the
// host-side status / last-error plumbing used by every extern "C" entry point.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

// ---------------------------------------------------------------------------
// Status codes returned by every C-ABI entry point (0 = success).
// ---------------------------------------------------------------------------
#define SKV_OK 0
#define SKV_ERR_BAD_ARG (-1)      // null pointer, non-positive size, mismatched shapes
#define SKV_ERR_UNSUPPORTED (-2)  // shape / dtype this build has no kernel for
#define SKV_ERR_WORKSPACE (-3)    // caller-provided workspace too small or misaligned
#define SKV_ERR_CUDA (-4)         // CUDA runtime / launch failure
#define SKV_ERR_DRIVER (-5)       // driver entry point (tensor-map encode) unavailable or failed

// KV storage types understood by the decode kernels.
#define SKV_KV_F16 0
#define SKV_KV_I8 1
#define SKV_KV_E4M3 2
#define SKV_OUT_BF16 0x100
#define SKV_V_INT4 0x200      // paged decode: V codes are 4-bit (mixed-precision page records)
#define SKV_EARLY_EXCEPT_LAST 0x400   // paged decode: only each sequence's last token is written by the previous kernel

// Bit set in the per-workspace device status word when a bounded wait gave up.
#define SKV_DEV_TIMEOUT 1
// Bit set when a page id read from a caller's page table lay outside the pools (the access was redirected or skipped).
#define SKV_DEV_BAD_PAGE 2

namespace skv {

// Thread-local message describing the last failure on this host thread.
inline char* last_error_buf() {
    static thread_local char buf[512] = {0};
    return buf;
}

inline int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(last_error_buf(), 512, fmt, ap);
    va_end(ap);
    return code;
}

#define SKV_CUDA_TRY(expr)                                                              \
    do {                                                                                \
        cudaError_t _e = (expr);                                                        \
        if (_e != cudaSuccess)                                                          \
            return ::skv::fail(SKV_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
    } while (0)

// RAII device switch: the reference launches on whatever device is current;
// here every entry point takes the device ordinal and restores the previous one.
struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
        if (dev != prev && cudaSetDevice(dev) != cudaSuccess) ok = false;
        target = dev;
    }
    ~DeviceGuard() {
        if (prev >= 0 && prev != target) cudaSetDevice(prev);
    }
    int target = -1;
};

inline int sm_count(int device) {
    static int cached[64] = {0};
    if (device >= 0 && device < 64 && cached[device] > 0) return cached[device];
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) n = 148;
    if (device >= 0 && device < 64) cached[device] = n;
    return n;
}

#if defined(__CUDACC__)
// Launch with the programmatic-stream-serialization attribute: if the previous kernel in the stream calls
// griddepcontrol.launch_dependents, this one may begin (its prologue and independent loads) before that
// kernel has drained; it must execute griddepcontrol.wait before touching anything that kernel writes.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// The same, with the CTAs of grid dimension y grouped into thread-block clusters of `cluster_y` (which must divide
// grid.y).  Sizes above 8 need cudaFuncAttributeNonPortableClusterSizeAllowed on the kernel.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                      int cluster_y, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 1;
    attr[1].val.clusterDim.y = (unsigned)cluster_y;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Plain launch (ordered like any other kernel) with the CTAs of grid dimension x grouped into clusters of `cluster_x`.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_cluster_x(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    int cluster_x, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cluster_x;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

template <typename... KArgs>
inline int max_active_clusters_x(void (*kernel)(KArgs...), dim3 block, size_t smem, int cluster_x) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)cluster_x, 1, 1);
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cluster_x;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

// How many clusters of `cluster_y` CTAs of this kernel the device can hold at once (0: such a launch would fail).
template <typename... KArgs>
inline int max_active_clusters(void (*kernel)(KArgs...), dim3 block, size_t smem, int cluster_y) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1, (unsigned)cluster_y, 1);
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = (unsigned)cluster_y;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}
#endif

// ---------------------------------------------------------------------------
// Device helpers
// ---------------------------------------------------------------------------
#if defined(__CUDACC__)

// A page id from a caller's table, made safe to turn into an address: an id outside [0, num_pages) becomes page 0
// and raises `bad`.  Branch-free on purpose -- a conditional atomic between two loads would pin their order and
// serialise a batch of gathers; the caller reports once, after its loads, with report_bad_page().  Never traps.
__device__ __forceinline__ int checked_page(int page, int num_pages, bool& bad) {
    const bool out_of_range = (unsigned)page >= (unsigned)num_pages;
    bad |= out_of_range;
    return out_of_range ? 0 : page;
}
__device__ __forceinline__ void report_bad_page(bool bad, int* status) {
    if (bad && status) atomicOr(status, SKV_DEV_BAD_PAGE);
}

// Range checks of data-dependent indices (instrumented builds only: -DSKV_BOUNDS).  compute-sanitizer stands in for
// nothing here, so the debug library checks itself: every index that is computed from data (a selected token or block,
// a page id, a list entry) goes through SKV_INDEX(i, n) before it becomes an address.  In the instrumented build an
// index outside [0, n) records the source line of the FIRST violation in a per-file device word, read back by that
// file's skv_debug_bounds_*(), and is replaced by 0 so that the access stays inside the buffer; nothing traps.  In the
// shipped build the macro is the index itself.
#ifdef SKV_BOUNDS
static __device__ int skv_bounds_word;   // one copy per translation unit; 0 = no violation seen
__device__ __forceinline__ long long skv_checked_index(long long i, long long n, int line) {
    if (i < 0 || i >= n) {
        atomicCAS(&skv_bounds_word, 0, line);
        return 0;
    }
    return i;
}
#define SKV_INDEX(i, n) ((int)::skv::skv_checked_index((long long)(i), (long long)(n), __LINE__))
#define SKV_BOUNDS_GETTER(name)                                                                            \
    extern "C" int name(int* out) {                                                                        \
        return cudaMemcpyFromSymbol(out, ::skv::skv_bounds_word, sizeof(int)) == cudaSuccess ? 0 : -4;     \
    }
#else
#define SKV_INDEX(i, n) (i)
#define SKV_BOUNDS_GETTER(name)
#endif

// Phase timestamps for kernel tuning (instrumented builds only: -DSKV_PROFILE_PHASES): thread 0 of CTA 0 records the
// global timer at numbered points; a per-file skv_debug_phase_ts_*() copies them out.  Compiled out of the shipped library.
#ifdef SKV_PROFILE_PHASES
static __device__ unsigned long long skv_phase_ts[32];   // one copy per translation unit
#define SKV_PHASE(i)                                                                   \
    do {                                                                               \
        if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0) { \
            unsigned long long t_;                                                     \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                     \
            skv_phase_ts[i] = t_;                                                      \
        }                                                                              \
    } while (0)
// the latest end of any CTA (slot 31; never reset: later launches end later)
#define SKV_PHASE_LAST_END()                                                           \
    do {                                                                               \
        if ((threadIdx.x & 31) == 0) {                                                 \
            unsigned long long t_;                                                     \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                     \
            atomicMax(&skv_phase_ts[31], t_);                                          \
        }                                                                              \
    } while (0)
#else
#define SKV_PHASE(i) do {} while (0)
#define SKV_PHASE_LAST_END() do {} while (0)
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Bounded wait on an mbarrier phase.  Returns false when the limit ran out, so
// that a mis-programmed copy turns into an error status instead of a hang.
#ifndef SKV_SPIN_LIMIT
#define SKV_SPIN_LIMIT (1u << 22)
#endif
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < SKV_SPIN_LIMIT; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tm) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tm)) : "memory");
}

// Every CTA fetches its own tile (no sharing of a load between the CTAs of a cluster).
// No cluster multicast: every CTA fetches its own tile.
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* tm, uint32_t bar,
                                            int c0, int c1, int c2, int c3, int c4, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4, %5, %6, %7}], [%2], %8;"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar),
          "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "l"(policy)
        : "memory");
}

// 4-D tiled TMA load (paged 8-bit pools).
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* tm, uint32_t bar,
                                            int c0, int c1, int c2, int c3, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4, %5, %6}], [%2], %7;"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar),
          "r"(c0), "r"(c1), "r"(c2), "r"(c3), "l"(policy)
        : "memory");
}

// 2-D tiled TMA load (weight and activation tiles of the skinny GEMM).  No cluster multicast.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int c0, int c1, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar), "r"(c0), "r"(c1), "l"(policy)
        : "memory");
}

__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

// Untiled bulk copy global -> shared (16-byte aligned addresses, size a multiple of 16).
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
        : "memory");
}

// Per-thread asynchronous copies global -> shared (Ampere-style cp.async): the data never occupies a register, so a
// thread can keep many of them in flight; completion is awaited by the issuing thread with cp_async_wait_all().
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.wait_all;" ::: "memory");
}

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

// D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col)
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col)
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Transpose an 8x8 matrix of 16-bit elements held in the MMA fragment layout (row r in lanes 4r..4r+3, two
// elements per lane): afterwards lane (g, tq) holds elements (2tq, g) and (2tq+1, g) of the original.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Programmatic dependent launch: let the next kernel in the stream start while this one is still running ...
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ... and, in that next kernel, wait until every earlier kernel has finished and its writes are visible.
__device__ __forceinline__ void pdl_wait_prior_grids() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// ---- thread-block clusters: rank, barrier, and loads from another CTA's shared memory ----
__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// Barrier over every thread of the cluster; all 32 lanes of a warp must reach it together.  Shared-memory writes made
// before it are visible to the other CTAs' loads after it.
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Address of this CTA's shared-memory location `local` in the CTA of rank `rank` of the same cluster.
__device__ __forceinline__ uint32_t cluster_map(uint32_t local, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    return remote;
}

__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

__device__ __forceinline__ float4 ld_cluster_f4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}

__device__ __forceinline__ float2 ld_cluster_f2(uint32_t addr) {
    float2 v;
    asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
    return v;
}

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// 16-byte streaming (evict-first) global load: data that is read exactly once.
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// Compiler fence on a loaded value: volatile asm statements keep their order, so everything that uses `v` after
// this call is scheduled after every load issued before it -- a batch of loads stays in flight together instead
// of being interleaved with (and serialised behind) the arithmetic on the first ones.
__device__ __forceinline__ void pin_loaded(uint4& v) {
    asm volatile("" : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w));
}

// fp32 dot product of 8 fp16 values (one 16-byte load) with 8 floats.
__device__ __forceinline__ float dot8(const uint4& kv, const float (&q)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&kv);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        s = fmaf(f.x, q[2 * i], s);
        s = fmaf(f.y, q[2 * i + 1], s);
    }
    return s;
}

// 8 fp16 values of a 16-byte word as floats.
__device__ __forceinline__ void unpack8(const uint4& raw, float (&x)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        x[2 * i] = f.x;
        x[2 * i + 1] = f.y;
    }
}

#endif  // __CUDACC__

}  // namespace skv
