// Tensor-parallel decode step: sum all-reduce of a [rows, hidden] activation over the GPUs of one node, fused with
// the residual add and the RMSNorm that consume it -- one kernel over NVLink peer memory instead of a library
// all-reduce (two kernels and ~15 us of latency for 128 KB) followed by a normalisation kernel.
//
// The reference is single-GPU (its model call is the Hugging Face module, benchmarks/llama_integration_benchmark.py:
// 266-279); this is the exchange step that KV-head sharding of the decode step adds after o_proj and down_proj.
//
// Protocol (every rank runs the same launches in the same order):
//   * each rank's GEMM writes its partial sum into its own buffer, which all peers can read (symmetric memory);
//   * the kernel's first CTA tells every peer "my partial of epoch e is complete" by storing e into slot [rank] of
//     the peer's flag array (release, system scope) -- at kernel start the GEMM before it in the stream is done;
//   * every CTA waits until all slots of its OWN flag array have reached e (acquire, system scope; BOUNDED: after
//     max_spins polls the kernel records SKV_DEV_TIMEOUT in its status word and stores nothing, and while the
//     status word is set later calls fail at once instead of waiting again);
//   * it then reads its row from all peers' partials, sums them in rank order in fp32 (so every rank gets the same
//     bits), rounds to the storage type, adds the residual stream in place and writes the normalised row;
//   * the epoch lives in device memory and is advanced by the last CTA, so a captured graph replays correctly.
// Two partial buffers alternate between consecutive calls: a rank overwrites a buffer only after it has passed the
// barrier of the call in between, which every peer reaches after it has finished reading that buffer.
// Only plain peer loads and stores are used.
#include <cuda_bf16.h>

#include "skv_common.cuh"

namespace skv {
namespace arn {

constexpr int THREADS = 256;
constexpr int MAX_RANKS = 8;

struct Peers {
    const uint16_t* partial[MAX_RANKS];   // rank r's [rows, hidden] partial sum
    uint32_t* flags[MAX_RANKS];           // rank r's flag array, MAX_RANKS words
};

template <typename T> struct Elem;
template <> struct Elem<__half> {
    static __device__ __forceinline__ float to_f(uint16_t b) { return __half2float(__ushort_as_half(b)); }
    static __device__ __forceinline__ uint16_t from_f(float x) { return __half_as_ushort(__float2half_rn(x)); }
};
template <> struct Elem<__nv_bfloat16> {
    static __device__ __forceinline__ float to_f(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }
    static __device__ __forceinline__ uint16_t from_f(float x) { return __bfloat16_as_ushort(__float2bfloat16_rn(x)); }
};

template <typename T>
__device__ __forceinline__ void unpack8h(const uint4& v, float (&x)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        x[2 * i] = Elem<T>::to_f((uint16_t)(w[i] & 0xFFFFu));
        x[2 * i + 1] = Elem<T>::to_f((uint16_t)(w[i] >> 16));
    }
}

template <typename T>
__device__ __forceinline__ uint4 pack8h(const float (&x)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = (uint32_t)Elem<T>::from_f(x[2 * i]) | ((uint32_t)Elem<T>::from_f(x[2 * i + 1]) << 16);
    return make_uint4(w[0], w[1], w[2], w[3]);
}

__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// 16 bytes of a peer's buffer, never served from this SM's L1
__device__ __forceinline__ uint4 ld_peer16(const void* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// sync words (this rank's own memory): [0] epoch of the last completed call, [1] ticket of the running call,
// [2] status (SKV_DEV_TIMEOUT when a wait ran out).  One CTA per row.
template <typename T, int WORLD, int MAXV>
__global__ void __launch_bounds__(THREADS)
allreduce_residual_rmsnorm_kernel(const Peers pp, uint32_t* sync, uint16_t* __restrict__ resid,
                                  const uint16_t* __restrict__ weight, uint16_t* __restrict__ out, int hidden, float eps,
                                  int rank, uint32_t max_spins) {
    __shared__ float red[THREADS / 32];
    __shared__ float bcast;
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(sync) + 1u;   // committed only after every CTA is done

    // The partial sums this flag announces were written by an EARLIER kernel of this stream (the GEMM), so they are
    // complete and visible to the peers before this kernel runs: the flag needs no fence in front of it, and a relaxed
    // system-scope store saves the one or two microseconds a system-wide fence costs on every call.
    if (blockIdx.x == 0 && tid < WORLD) st_relaxed_sys(pp.flags[tid] + rank, epoch);
    // Once a wait has run out the status word stays set and later calls do not wait again: a dead peer costs one
    // bounded wait, not one per call.
    const bool failed_before = *reinterpret_cast<volatile uint32_t*>(sync + 2) != 0u;
    bool arrived = true;
    if (tid < WORLD) {
        arrived = false;
        const uint32_t* slot = pp.flags[rank] + tid;
        for (uint32_t i = 0; i < (failed_before ? 0u : max_spins); ++i) {
            if ((int32_t)(ld_acquire_sys(slot) - epoch) >= 0) { arrived = true; break; }
            __nanosleep(64);
        }
    }
    const bool all_arrived = __syncthreads_and(arrived);

    if (all_arrived) {
        const long long base = (long long)row * hidden;
        float x[MAXV][8];
        float ss = 0.f;
        uint4 part[MAXV][WORLD];
#pragma unroll
        for (int v = 0; v < MAXV; ++v) {
            const int c = min((v * THREADS + tid) * 8, hidden - 8);   // clamped: loads need no condition
#pragma unroll
            for (int r = 0; r < WORLD; ++r) part[v][r] = ld_peer16(pp.partial[r] + base + c);
        }
#pragma unroll
        for (int v = 0; v < MAXV; ++v) {
            const int c = (v * THREADS + tid) * 8;
            if (c < hidden) {
                float acc[8];
                unpack8h<T>(part[v][0], acc);
#pragma unroll
                for (int r = 1; r < WORLD; ++r) {
                    float d[8];
                    unpack8h<T>(part[v][r], d);
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[i] += d[i];
                }
                unpack8h<T>(*reinterpret_cast<const uint4*>(resid + base + c), x[v]);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float delta = Elem<T>::to_f(Elem<T>::from_f(acc[i]));          // the all-reduced value, rounded
                    x[v][i] = Elem<T>::to_f(Elem<T>::from_f(x[v][i] + delta));         // the residual stream, rounded
                }
                *reinterpret_cast<uint4*>(resid + base + c) = pack8h<T>(x[v]);
#pragma unroll
                for (int i = 0; i < 8; ++i) ss = fmaf(x[v][i], x[v][i], ss);
            }
        }
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        if (warp == 0) {
            float t = lane < THREADS / 32 ? red[lane] : 0.f;
            t = warp_sum(t);
            if (lane == 0) bcast = rsqrtf(t / (float)hidden + eps);
        }
        __syncthreads();
        const float inv = bcast;
#pragma unroll
        for (int v = 0; v < MAXV; ++v) {
            const int c = (v * THREADS + tid) * 8;
            if (c < hidden) {
                float w[8], y[8];
                unpack8h<T>(*reinterpret_cast<const uint4*>(weight + c), w);
#pragma unroll
                for (int i = 0; i < 8; ++i) y[i] = x[v][i] * inv * w[i];
                *reinterpret_cast<uint4*>(out + base + c) = pack8h<T>(y);
            }
        }
    } else if (tid == 0) {
        atomicOr(reinterpret_cast<int*>(sync + 2), SKV_DEV_TIMEOUT);
    }

    // the last CTA to finish advances the epoch (also after a timeout, so that later calls stay in step)
    __syncthreads();
    if (tid == 0) {
        const uint32_t t = atomicAdd(sync + 1, 1u);
        if (t == gridDim.x - 1) {
            sync[1] = 0u;
            __threadfence();
            *reinterpret_cast<volatile uint32_t*>(sync) = epoch;
        }
    }
}

template <typename T, int WORLD>
static void launch(const Peers& pp, uint32_t* sync, uint16_t* resid, const uint16_t* weight, uint16_t* out, int rows,
                   int hidden, float eps, int rank, uint32_t max_spins, cudaStream_t st) {
    if (hidden <= THREADS * 8 * 2)
        allreduce_residual_rmsnorm_kernel<T, WORLD, 2><<<rows, THREADS, 0, st>>>(pp, sync, resid, weight, out, hidden, eps, rank, max_spins);
    else
        allreduce_residual_rmsnorm_kernel<T, WORLD, 4><<<rows, THREADS, 0, st>>>(pp, sync, resid, weight, out, hidden, eps, rank, max_spins);
}

template <typename T>
static int dispatch(int world, const Peers& pp, uint32_t* sync, uint16_t* resid, const uint16_t* weight, uint16_t* out,
                    int rows, int hidden, float eps, int rank, uint32_t max_spins, cudaStream_t st) {
    switch (world) {
        case 1: launch<T, 1>(pp, sync, resid, weight, out, rows, hidden, eps, rank, max_spins, st); break;
        case 2: launch<T, 2>(pp, sync, resid, weight, out, rows, hidden, eps, rank, max_spins, st); break;
        case 4: launch<T, 4>(pp, sync, resid, weight, out, rows, hidden, eps, rank, max_spins, st); break;
        case 8: launch<T, 8>(pp, sync, resid, weight, out, rows, hidden, eps, rank, max_spins, st); break;
        default: return fail(SKV_ERR_UNSUPPORTED, "world size %d not supported (1, 2, 4 or 8)", world);
    }
    return SKV_OK;
}

}  // namespace arn
}  // namespace skv

using namespace skv;

extern "C" {

int skv_allreduce_residual_rmsnorm(const void* const* peer_partials, void* const* peer_flags, void* sync_words,
                                   void* resid, const void* weight, void* out, int rows, int hidden, float eps,
                                   int is_bf16, int rank, int world, unsigned max_spins, int device, void* stream) {
    if (!peer_partials || !peer_flags || !sync_words || !resid || !weight || !out)
        return fail(SKV_ERR_BAD_ARG, "skv_allreduce_residual_rmsnorm: null pointer");
    if (world < 1 || world > arn::MAX_RANKS || rank < 0 || rank >= world)
        return fail(SKV_ERR_BAD_ARG, "rank %d outside world of %d (at most %d)", rank, world, arn::MAX_RANKS);
    if (rows <= 0 || rows > 65535 || hidden < 8 || hidden % 8) return fail(SKV_ERR_BAD_ARG, "rows must be in 1..65535 and hidden a positive multiple of 8");
    if (hidden > arn::THREADS * 8 * 4) return fail(SKV_ERR_UNSUPPORTED, "hidden %d exceeds %d", hidden, arn::THREADS * 8 * 4);
    if (max_spins == 0) return fail(SKV_ERR_BAD_ARG, "max_spins must be positive");
    arn::Peers pp;
    for (int r = 0; r < arn::MAX_RANKS; ++r) {
        const int s = r < world ? r : world - 1;
        if (!peer_partials[s] || !peer_flags[s]) return fail(SKV_ERR_BAD_ARG, "null peer pointer for rank %d", s);
        if ((reinterpret_cast<uintptr_t>(peer_partials[s]) & 15) || (reinterpret_cast<uintptr_t>(peer_flags[s]) & 3))
            return fail(SKV_ERR_BAD_ARG, "peer buffers must be 16-byte aligned");
        pp.partial[r] = static_cast<const uint16_t*>(peer_partials[s]);
        pp.flags[r] = static_cast<uint32_t*>(peer_flags[s]);
    }
    if ((reinterpret_cast<uintptr_t>(resid) | reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(out)) & 15)
        return fail(SKV_ERR_BAD_ARG, "skv_allreduce_residual_rmsnorm: tensors must be 16-byte aligned");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(SKV_ERR_CUDA, "cannot switch to device %d", device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    auto* sy = static_cast<uint32_t*>(sync_words);
    auto* rs = static_cast<uint16_t*>(resid);
    auto* w = static_cast<const uint16_t*>(weight);
    auto* o = static_cast<uint16_t*>(out);
    const int rc = is_bf16 ? arn::dispatch<__nv_bfloat16>(world, pp, sy, rs, w, o, rows, hidden, eps, rank, max_spins, st)
                           : arn::dispatch<__half>(world, pp, sy, rs, w, o, rows, hidden, eps, rank, max_spins, st);
    if (rc) return rc;
    SKV_CUDA_TRY(cudaGetLastError());
    return SKV_OK;
}

}  // extern "C"
