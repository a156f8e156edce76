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

// ---------------------------------------------------------------------------------------------------------------
// Push variant.  The pull protocol above costs two NVLink traversals in sequence (the flag to the peer, then the
// peer's loads of the data and their way back).  Here every rank WRITES its partial row into a receive buffer of every
// peer, and the data carries its own flag: an 8-byte word holds 4 bytes of the partial (two 16-bit values) and the
// 32-bit epoch of the call, and an aligned 8-byte store arrives whole -- no flag array, no fence, one traversal.  The
// receiver polls its OWN memory until every word of its row shows the call's epoch (bounded, as above), then sums the
// ranks' contributions in rank order (its own from registers), so all ranks compute the same bits.
//   receive region of a rank, per call parity: [world (source rank)][rows][hidden / 2] words of 8 bytes;
//   pp.recv[r] is rank r's region for this call's parity.  Zero-filled before the first call; epochs start at 1.
// A buffer is rewritten two calls later, which a rank reaches only after every peer has passed the call in between
// and therefore finished reading -- the same argument as for the two partial buffers above.
// ---------------------------------------------------------------------------------------------------------------
struct PushPeers {
    uint8_t* recv[MAX_RANKS];
};

__device__ __forceinline__ void st_ll16(void* p, uint32_t d0, uint32_t d1, uint32_t epoch) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(d0), "r"(epoch), "r"(d1), "r"(epoch) : "memory");
}

template <typename T, int WORLD, int MAXV>
__global__ void __launch_bounds__(THREADS)
allreduce_push_residual_rmsnorm_kernel(const PushPeers pp, const uint16_t* __restrict__ partial, uint32_t* sync,
                                       uint16_t* __restrict__ resid, const uint16_t* __restrict__ weight,
                                       uint16_t* __restrict__ out, int hidden, float eps, int rank, uint32_t max_spins) {
    __shared__ float red[THREADS / 32];
    __shared__ float bcast;
    const int row = blockIdx.x, rows = gridDim.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(sync) + 1u;   // committed only after every CTA is done
    const bool failed_before = *reinterpret_cast<volatile uint32_t*>(sync + 2) != 0u;
    const long long base = (long long)row * hidden;

    // this rank's partial row (written by an earlier kernel of the stream), pushed to every peer with the epoch
    uint4 mine[MAXV];
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
        const int c = (v * THREADS + tid) * 8;
        mine[v] = make_uint4(0u, 0u, 0u, 0u);
        if (c < hidden) {
            mine[v] = *reinterpret_cast<const uint4*>(partial + base + c);
            const long long off = (((long long)rank * rows + row) * hidden + c) * 4;   // 8-byte words: 4 bytes per element pair... 4 bytes of buffer per element
#pragma unroll
            for (int r = 0; r < WORLD; ++r) {
                if (r == rank) continue;
                st_ll16(pp.recv[r] + off, mine[v].x, mine[v].y, epoch);
                st_ll16(pp.recv[r] + off + 16, mine[v].z, mine[v].w, epoch);
            }
        }
    }

    // the peers' rows, from this rank's own receive region: every poll round issues the loads of all words still
    // missing back to back (one trip to L2 per round, not one per word)
    uint4 part[MAXV][WORLD];
    uint32_t pending = 0u;
#pragma unroll
    for (int v = 0; v < MAXV; ++v)
#pragma unroll
        for (int r = 0; r < WORLD; ++r) {
            part[v][r] = mine[v];
            if (r != rank && (v * THREADS + tid) * 8 < hidden) pending |= 1u << (v * WORLD + r);
        }
    for (uint32_t spin = 0; pending != 0u && spin < (failed_before ? 0u : max_spins); ++spin) {
        uint4 wa[MAXV][WORLD], wb[MAXV][WORLD];
#pragma unroll
        for (int v = 0; v < MAXV; ++v)
#pragma unroll
            for (int r = 0; r < WORLD; ++r)
                if (pending & (1u << (v * WORLD + r))) {
                    const uint8_t* src = pp.recv[rank] + (((long long)r * rows + row) * hidden + (v * THREADS + tid) * 8) * 4;
                    wa[v][r] = ld_peer16(src);
                    wb[v][r] = ld_peer16(src + 16);
                }
#pragma unroll
        for (int v = 0; v < MAXV; ++v)
#pragma unroll
            for (int r = 0; r < WORLD; ++r)
                if (pending & (1u << (v * WORLD + r))) {
                    const uint4 a = wa[v][r], b = wb[v][r];
                    if (a.y == epoch && a.w == epoch && b.y == epoch && b.w == epoch) {
                        part[v][r] = make_uint4(a.x, a.z, b.x, b.z);
                        pending &= ~(1u << (v * WORLD + r));
                    }
                }
    }
    const bool arrived = pending == 0u;
    const bool all_arrived = __syncthreads_and(arrived);

    if (all_arrived) {
        float x[MAXV][8];
        float ss = 0.f;
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
static void launch_push(const PushPeers& pp, const uint16_t* partial, uint32_t* sync, uint16_t* resid, const uint16_t* weight,
                        uint16_t* out, int rows, int hidden, float eps, int rank, uint32_t max_spins, cudaStream_t st) {
    // (rows wider than 4096 elements would need 4 vectors per thread: at 8 ranks their words in flight no longer fit
    // the register file, so wider rows are left to the pull protocol)
    allreduce_push_residual_rmsnorm_kernel<T, WORLD, 2><<<rows, THREADS, 0, st>>>(pp, partial, sync, resid, weight, out, hidden, eps, rank, max_spins);
}

template <typename T>
static int dispatch_push(int world, const PushPeers& pp, const uint16_t* partial, uint32_t* sync, uint16_t* resid,
                         const uint16_t* weight, uint16_t* out, int rows, int hidden, float eps, int rank, uint32_t max_spins,
                         cudaStream_t st) {
    switch (world) {
        case 1: launch_push<T, 1>(pp, partial, sync, resid, weight, out, rows, hidden, eps, rank, max_spins, st); break;
        case 2: launch_push<T, 2>(pp, partial, sync, resid, weight, out, rows, hidden, eps, rank, max_spins, st); break;
        case 4: launch_push<T, 4>(pp, partial, sync, resid, weight, out, rows, hidden, eps, rank, max_spins, st); break;
        case 8: launch_push<T, 8>(pp, partial, sync, resid, weight, out, rows, hidden, eps, rank, max_spins, st); break;
        default: return fail(SKV_ERR_UNSUPPORTED, "world size %d not supported (1, 2, 4 or 8)", world);
    }
    return SKV_OK;
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

// Push variant (see allreduce_push_residual_rmsnorm_kernel): `partial` is this rank's [rows, hidden] partial sum in its
// own memory; peer_recv[r] is the device address, valid on THIS GPU, of rank r's receive region for this call's parity
// ([world][rows][hidden / 2] 8-byte words, zero-filled before the first call; consecutive calls alternate between two
// regions).  sync_words as for skv_allreduce_residual_rmsnorm.
int skv_allreduce_residual_rmsnorm_push(const void* partial, void* const* peer_recv, void* sync_words, void* resid,
                                        const void* weight, void* out, int rows, int hidden, float eps, int is_bf16,
                                        int rank, int world, unsigned max_spins, int device, void* stream) {
    if (!partial || !peer_recv || !sync_words || !resid || !weight || !out)
        return fail(SKV_ERR_BAD_ARG, "skv_allreduce_residual_rmsnorm_push: null pointer");
    if (world < 1 || world > arn::MAX_RANKS || rank < 0 || rank >= world)
        return fail(SKV_ERR_BAD_ARG, "rank %d / world %d out of range (at most %d ranks)", rank, world, arn::MAX_RANKS);
    if (rows <= 0 || rows > 65535 || hidden <= 0 || hidden % 8 || hidden > arn::THREADS * 8 * 2)
        return fail(SKV_ERR_UNSUPPORTED, "rows must be in 1..65535 and hidden a multiple of 8 up to %d (got %d x %d)",
                    arn::THREADS * 8 * 2, rows, hidden);
    arn::PushPeers pp;
    for (int r = 0; r < arn::MAX_RANKS; ++r) {
        const int s = r < world ? r : 0;
        if (!peer_recv[s]) return fail(SKV_ERR_BAD_ARG, "null receive region for rank %d", s);
        if (reinterpret_cast<uintptr_t>(peer_recv[s]) & 15) return fail(SKV_ERR_BAD_ARG, "receive regions must be 16-byte aligned");
        pp.recv[r] = static_cast<uint8_t*>(peer_recv[s]);
    }
    if ((reinterpret_cast<uintptr_t>(partial) | reinterpret_cast<uintptr_t>(resid) | reinterpret_cast<uintptr_t>(weight) |
         reinterpret_cast<uintptr_t>(out)) & 15)
        return fail(SKV_ERR_BAD_ARG, "skv_allreduce_residual_rmsnorm_push: tensors must be 16-byte aligned");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(SKV_ERR_CUDA, "cannot switch to device %d", device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    auto* pa = static_cast<const uint16_t*>(partial);
    auto* sy = static_cast<uint32_t*>(sync_words);
    auto* rs = static_cast<uint16_t*>(resid);
    auto* w = static_cast<const uint16_t*>(weight);
    auto* o = static_cast<uint16_t*>(out);
    const int rc = is_bf16 ? arn::dispatch_push<__nv_bfloat16>(world, pp, pa, sy, rs, w, o, rows, hidden, eps, rank, max_spins, st)
                           : arn::dispatch_push<__half>(world, pp, pa, sy, rs, w, o, rows, hidden, eps, rank, max_spins, st);
    if (rc) return rc;
    SKV_CUDA_TRY(cudaGetLastError());
    return SKV_OK;
}

}  // extern "C"
