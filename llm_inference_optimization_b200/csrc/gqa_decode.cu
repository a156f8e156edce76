// Dense grouped-query decode attention for one new token per sequence, split
// over the KV length so that every SM streams a share of the cache, with the
// log-sum-exp combine done by the last CTA to finish each (batch, kv-head).
//
// Replaces gqa_decode_kernel / launch_fused_gqa of the reference
// (csrc/kernels/gqa_decode.cu:84-215, :218-290), which runs one CTA per query
// head (re-reading the KV of a group once per query head) with no KV split.
//
//   Out[b, hq, :] = softmax(scale * Q[b, hq, :] . K[b, :, hq / G, :]^T) . V[b, :, hq / G, :]
//
// Mapping to the hardware:
//   * grid (Hkv, splits, B): a CTA owns one kv-head of one sequence over a
//     contiguous token range and serves all G = Hq / Hkv query heads of the
//     group, so each K/V byte is read from HBM exactly once.
//   * one producer warp issues TMA tile loads (cp.async.bulk.tensor, 128-byte
//     swizzle, L2 evict-first) into a ring of shared-memory stages guarded by
//     full/empty mbarriers; four consumer warps each take 16 tokens of every
//     64-token stage.
//   * the group x tile products run on the tensor cores as mma.sync m16n8k16
//     with the query group on the M dimension (rows >= G are zero padding):
//     S = Q K^T with K fragments read by ldmatrix, P V with V fragments read by
//     ldmatrix.trans.  Softmax is online, fp32, in the exp2 domain.
//   * every warp keeps its own (max, sum, O) state; warps are merged through
//     shared memory, splits through an fp32 workspace and an atomic ticket.
//   * every mbarrier wait is bounded; a wait that runs out sets a bit in the
//     workspace status word instead of hanging.
#include <mutex>

#include "gqa_epilogue.cuh"
#include "skv_common.cuh"
#include "skv_tmap.cuh"

namespace skv {
namespace gqa {

struct Params {
    const __half* q;
    __half* out;
    float* partial_o;    // [B, Hkv, S, G, D]
    float* partial_ml;   // [B, Hkv, S, G, 2]  (running max in the exp2 domain, running sum)
    int* tickets;        // [B * Hkv], zero between launches
    int* status;         // device status word
    const int* seq_lens; // [B] or null
    int N, Hq, Hkv, G;
    int tiles_per_split, num_splits, stages;
    int list_items, B;   // list_items > 0: grid (Hkv, list_items), work-list schedule of a ragged batch (worklist_item)
    int cluster_combine; // 1: launched with clusters of num_splits CTAs along y; splits are summed through shared memory
    long long q_stride_b, q_stride_h, o_stride_b, o_stride_h;
    float scale_log2;    // softmax scale * log2(e)
    int early_kv;        // K/V and seq_lens are not produced by the previous kernel: stream them before it completes
    float* score_out;    // optional [B, Hq, N] fp32: scaled scores in the exp2 domain, for the attention-mass pass
    float* ml_final;     // optional [B, Hq, 2]: final softmax maximum and denominator per head
    KvMapPos pos;
};

template <int D>
struct Smem {
    static constexpr int NH = D / 64;                 // 128-byte halves per row
    static constexpr int HALF_BYTES = TILE * 128;     // one [TILE][64] fp16 block
    static constexpr int KV_BYTES = NH * HALF_BYTES;  // K (or V) part of a stage
    static constexpr int STAGE_BYTES = 2 * KV_BYTES;
    static size_t bytes(int stages) {
        size_t ring = (size_t)stages * STAGE_BYTES;
        size_t merge = epilogue_smem_bytes<D>();
        size_t body = ring > merge ? ring : merge;
        return 1024 /*alignment slack*/ + body + 2 * stages * 8 + 16;
    }
};

__device__ __forceinline__ void kv_tile_load(uint32_t dst, const CUtensorMap* tm, uint32_t bar, const KvMapPos& pos,
                                             int half, int tok, int head, int batch, uint64_t policy) {
    int c[5] = {0, 0, 0, 0, 0};
#pragma unroll
    for (int i = 1; i < 5; ++i)
        c[i] = (i == pos.half) ? half : (i == pos.tok) ? tok : (i == pos.head) ? head : batch;
    tma_load_5d(dst, tm, bar, c[0], c[1], c[2], c[3], c[4], policy);
}

template <int D>
__global__ void __launch_bounds__(THREADS, 1)
gqa_decode_f16_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                      const Params p) {
    using S = Smem<D>;
    constexpr int KSTEPS = D / 16;  // MMA k-steps across the head dimension
    constexpr int NT_O = D / 8;     // 8-channel output tiles

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.x;
    int split = blockIdx.y, b = blockIdx.z;

    // Launched with programmatic stream serialisation, this kernel may start before the previous one in the stream
    // has completed.  By default every thread waits for it here, so the kernel is ordered like any other; only when
    // the caller has declared that K, V and seq_lens are not produced by the previous kernel (early_kv) does the
    // wait move down to the consumers, and the producer streams K/V meanwhile.
    SKV_PHASE(0);
    if (!p.early_kv) pdl_wait_prior_grids();
    int len, n_splits, tiles_per_split = p.tiles_per_split;
    if (p.list_items > 0) {   // work-list schedule of a ragged batch (see worklist_item)
        const SplitItem it = worklist_item(p.seq_lens, p.B, p.N, p.list_items, blockIdx.y, p.tiles_per_split);
        if (it.b < 0) return;
        b = it.b; split = it.split; len = it.len; n_splits = it.n_splits; tiles_per_split = it.tiles_per_split;
    } else {
        len = p.seq_lens ? min(max(p.seq_lens[b], 0), p.N) : p.N;
        const int tps_tokens = tiles_per_split * TILE;
        n_splits = len > 0 ? (len + tps_tokens - 1) / tps_tokens : 1;
        if (split >= n_splits) {
            if (p.cluster_combine) {   // nothing to add, but every thread of a cluster passes both of its barriers
                cluster_barrier();
                cluster_barrier();
            }
            return;
        }
    }
    const int tokens_per_split = tiles_per_split * TILE;
    const int t_begin = split * tokens_per_split;
    const int t_end = min(len, t_begin + tokens_per_split);
    const int ntiles = (t_end - t_begin + TILE - 1) / TILE;  // 0 for an empty sequence

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t ring = smem_u32(smem);
    size_t body = (size_t)p.stages * S::STAGE_BYTES;
    if (epilogue_smem_bytes<D>() > body) body = epilogue_smem_bytes<D>();
    const uint32_t full_bar = ring + (uint32_t)body;
    const uint32_t empty_bar = full_bar + p.stages * 8;
    int* last_flag = reinterpret_cast<int*>(smem + body + 2 * p.stages * 8);

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(full_bar + s * 8, 1);
            mbar_init(empty_bar + s * 8, CONSUMER_WARPS);
        }
        fence_barrier_init();
    }
    __syncthreads();
    SKV_PHASE(1);
    // ------------------------------------------------------------------ producer
    if (warp == CONSUMER_WARPS) {
        if (lane == 0) {
            tma_prefetch_desc(&tmK);
            tma_prefetch_desc(&tmV);
            const uint64_t policy = l2_policy_evict_first();
            int s = 0;        // stage and ring-pass phase advance incrementally: no divisions in this loop
            uint32_t ph = 0;
            for (int it = 0; it < ntiles; ++it, ++s) {
                if (s == p.stages) { s = 0; ph ^= 1u; }
                if (it >= p.stages && !mbar_wait(empty_bar + s * 8, ph ^ 1u)) {
                    atomicOr(p.status, SKV_DEV_TIMEOUT);
                    break;
                }
                const uint32_t bar = full_bar + s * 8;
                mbar_expect_tx(bar, S::STAGE_BYTES);
                const int tok = t_begin + it * TILE;
                const uint32_t kdst = ring + s * S::STAGE_BYTES;
#pragma unroll
                for (int hf = 0; hf < S::NH; ++hf) {
                    kv_tile_load(kdst + hf * S::HALF_BYTES, &tmK, bar, p.pos, hf, tok, h, b, policy);
                    kv_tile_load(kdst + S::KV_BYTES + hf * S::HALF_BYTES, &tmV, bar, p.pos, hf, tok, h, b, policy);
                }
            }
        }
        if (p.cluster_combine) {
            __syncwarp();
            cluster_barrier();
            cluster_barrier();
        }
        return;
    }

    // ----------------------------------------------------------------- consumers
    const int g = lane >> 2;   // MMA row (query head within the group); rows g and g + 8
    const int tq = lane & 3;   // column pair within an 8-wide tile
    const int G = p.G;

    // The query may be the previous kernel's output and the workspace / output written below certainly depend on
    // it: in early_kv mode the wait is here.  Only after it is the NEXT launch released (it may start its prologue,
    // and in early_kv mode its K/V stream, as SMs free up): a kernel released at this point starts after
    // everything older than this kernel has completed, and this kernel itself never writes K or V.
    if (p.early_kv) pdl_wait_prior_grids();
    pdl_launch_dependents();

    // Query fragments for all k-steps, zero for padding rows.
    uint32_t qa[KSTEPS][4];
    {
        const __half* q0 = p.q + (long long)b * p.q_stride_b + (long long)(h * G + g) * p.q_stride_h;
        const __half* q1 = q0 + 8 * p.q_stride_h;
        const bool v0 = g < G, v1 = g + 8 < G;
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {
            const int col = kk * 16 + tq * 2;
            qa[kk][0] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + col) : 0u;
            qa[kk][1] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + col) : 0u;
            qa[kk][2] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + col + 8) : 0u;
            qa[kk][3] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + col + 8) : 0u;
        }
    }

    float o[NT_O][4];
#pragma unroll
    for (int n = 0; n < NT_O; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY;  // running max (exp2 domain), rows g / g + 8
    float l0 = 0.f, l1 = 0.f;              // per-thread partial row sums

    // ldmatrix lane roles: matrix j = lane / 8, row r8 = lane % 8.
    const int lj = lane >> 3, r8 = lane & 7;
    const int wtok = warp * 16;  // this warp's first token inside a stage

    int s = 0;
    uint32_t ph = 0;
    SKV_PHASE(2);
    for (int it = 0; it < ntiles; ++it, ++s) {
        if (s == p.stages) { s = 0; ph ^= 1u; }
        if (!mbar_wait(full_bar + s * 8, ph)) {
            if (lane == 0) atomicOr(p.status, SKV_DEV_TIMEOUT);
            break;
        }
        if (it == 0) SKV_PHASE(3);
        const int tok0 = t_begin + it * TILE + wtok;  // global index of this warp's first token
        if (tok0 < t_end) {
            const uint32_t kbase = ring + s * S::STAGE_BYTES;
            const uint32_t vbase = kbase + S::KV_BYTES;

            // ---- S = Q K^T for 16 tokens: two 8-token tiles
            float sc[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
#pragma unroll
            for (int kk2 = 0; kk2 < KSTEPS / 2; ++kk2) {
                const int c = 4 * kk2 + lj;  // 16-byte chunk of the row
                const uint32_t coff = (uint32_t)(c >> 3) * S::HALF_BYTES + (uint32_t)(((c & 7) ^ r8) << 4);
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    const uint32_t row = (uint32_t)(wtok + nt * 8 + r8);
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4(kbase + row * 128 + coff, b0, b1, b2, b3);
                    mma_f16(sc[nt], qa[2 * kk2], b0, b1);
                    mma_f16(sc[nt], qa[2 * kk2 + 1], b2, b3);
                }
            }

            // ---- scale into the exp2 domain, mask the ragged end of the sequence
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) sc[nt][j] *= p.scale_log2;
            if (tok0 + 16 > t_end) {
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (tok0 + nt * 8 + tq * 2 + (j & 1) >= t_end) sc[nt][j] = -INFINITY;
            }

            // ---- optional: keep the scores, so that a second pass can turn them into attention probabilities once
            //      the softmax maximum and denominator of the whole sequence are known
            if (p.score_out) {
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    const int t = tok0 + nt * 8 + tq * 2;
                    if (g < G) {
                        float* d0 = p.score_out + ((long long)b * p.Hq + h * G + g) * p.N + t;
                        if (t < t_end) d0[0] = sc[nt][0];
                        if (t + 1 < t_end) d0[1] = sc[nt][1];
                    }
                    if (g + 8 < G) {
                        float* d1 = p.score_out + ((long long)b * p.Hq + h * G + g + 8) * p.N + t;
                        if (t < t_end) d1[0] = sc[nt][2];
                        if (t + 1 < t_end) d1[1] = sc[nt][3];
                    }
                }
            }

            // ---- online softmax
            float mx0 = fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[1][0], sc[1][1]));
            float mx1 = fmaxf(fmaxf(sc[0][2], sc[0][3]), fmaxf(sc[1][2], sc[1][3]));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
            if (__any_sync(0xffffffffu, (mn0 > m0) || (mn1 > m1))) {
                const float c0 = fast_exp2(m0 - mn0), c1 = fast_exp2(m1 - mn1);
                l0 *= c0;
                l1 *= c1;
#pragma unroll
                for (int n = 0; n < NT_O; ++n) {
                    o[n][0] *= c0; o[n][1] *= c0;
                    o[n][2] *= c1; o[n][3] *= c1;
                }
                m0 = mn0;
                m1 = mn1;
            }
            uint32_t pa[4];
            {
                const float p00 = fast_exp2(sc[0][0] - m0), p01 = fast_exp2(sc[0][1] - m0);
                const float p02 = fast_exp2(sc[0][2] - m1), p03 = fast_exp2(sc[0][3] - m1);
                const float p10 = fast_exp2(sc[1][0] - m0), p11 = fast_exp2(sc[1][1] - m0);
                const float p12 = fast_exp2(sc[1][2] - m1), p13 = fast_exp2(sc[1][3] - m1);
                l0 += (p00 + p01) + (p10 + p11);
                l1 += (p02 + p03) + (p12 + p13);
                pa[0] = pack_half2(p00, p01);
                pa[1] = pack_half2(p02, p03);
                pa[2] = pack_half2(p10, p11);
                pa[3] = pack_half2(p12, p13);
            }

            // ---- rows past the end of the sequence may hold anything (even NaN): zero them in V
            if (tok0 + 16 > t_end) {
                for (int idx = lane; idx < 16 * (D / 8); idx += 32) {
                    const int r = idx / (D / 8), c = idx - r * (D / 8);
                    if (tok0 + r >= t_end)
                        *reinterpret_cast<uint4*>(smem + (size_t)s * S::STAGE_BYTES + S::KV_BYTES +
                                                  (size_t)(c >> 3) * S::HALF_BYTES + (size_t)(wtok + r) * 128 +
                                                  (size_t)(c & 7) * 16) = make_uint4(0u, 0u, 0u, 0u);
                }
                __syncwarp();
            }

            // ---- O += P V over the 16 tokens
#pragma unroll
            for (int np = 0; np < NT_O / 2; ++np) {
                const int c = 2 * np + (lj >> 1);
                const uint32_t row = (uint32_t)(wtok + (lj & 1) * 8 + r8);
                const uint32_t addr = vbase + (uint32_t)(c >> 3) * S::HALF_BYTES + row * 128 +
                                      (uint32_t)(((c & 7) ^ r8) << 4);
                uint32_t b0, b1, b2, b3;
                ldsm_x4_t(addr, b0, b1, b2, b3);
                mma_f16(o[2 * np], pa, b0, b1);
                mma_f16(o[2 * np + 1], pa, b2, b3);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar + s * 8);
    }

    // ------------------------------------------------- merge the four warps
    SKV_PHASE(4);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

    named_bar_sync(1, CONSUMER_THREADS);  // every stage is drained: the ring can be reused
    float* mo = reinterpret_cast<float*>(smem);                          // [W][MAX_GROUP][D]
    float* mm = mo + CONSUMER_WARPS * MAX_GROUP * D;                     // [W][MAX_GROUP]
    float* ml = mm + CONSUMER_WARPS * MAX_GROUP;                         // [W][MAX_GROUP]
    {
        float* my = mo + (warp * MAX_GROUP) * D;
        if (g < G) {
#pragma unroll
            for (int n = 0; n < NT_O; ++n)
                *reinterpret_cast<float2*>(my + g * D + n * 8 + tq * 2) = make_float2(o[n][0], o[n][1]);
            if (tq == 0) { mm[warp * MAX_GROUP + g] = m0; ml[warp * MAX_GROUP + g] = l0; }
        }
        if (g + 8 < G) {
#pragma unroll
            for (int n = 0; n < NT_O; ++n)
                *reinterpret_cast<float2*>(my + (g + 8) * D + n * 8 + tq * 2) = make_float2(o[n][2], o[n][3]);
            if (tq == 0) { mm[warp * MAX_GROUP + g + 8] = m1; ml[warp * MAX_GROUP + g + 8] = l1; }
        }
    }
    named_bar_sync(1, CONSUMER_THREADS);
    EpilogueArgs ea;
    ea.partial_o = p.partial_o; ea.partial_ml = p.partial_ml; ea.tickets = p.tickets; ea.out = p.out;
    ea.Hkv = p.Hkv; ea.G = G; ea.num_splits = p.num_splits; ea.o_stride_b = p.o_stride_b; ea.o_stride_h = p.o_stride_h;
    ea.ml_final = p.ml_final;
    if (p.cluster_combine) {
        // The splits of this (b, h) are the CTAs of one cluster (rank == split): each leaves its merged result in its
        // own shared memory, rank 0 sums them through distributed shared memory, and nobody leaves before it has.
        SKV_PHASE(5);
        cluster_merge_publish<D>(smem, G, 1.f);
        SKV_PHASE(6);
        cluster_barrier();
        SKV_PHASE(7);
        if (cluster_cta_rank() == 0) cluster_combine_rank0<D>(ea, smem, b, h, n_splits);
        SKV_PHASE(8);
        cluster_barrier();
        SKV_PHASE(9);
        return;
    }
    SKV_PHASE(5);
    merge_and_combine<D>(ea, smem, last_flag, b, h, split, n_splits, 1.f);
    SKV_PHASE(9);
    SKV_PHASE_LAST_END();
}

// Attention mass of every cached token, summed over the query heads of its group and ADDED to `mass`:
//   mass[b, hkv, t] += sum_g exp2(score[b, hkv*G+g, t] - M[b, hkv*G+g]) / L[b, hkv*G+g]
// -- the running importance score an eviction policy keeps per token (the `scores` argument of the reference's
// fused_kv_evict, sparse_kv/eviction.py:12-22, which the reference leaves to the caller to produce).
// grid (ceil(N / 256), Hkv, B)
__global__ void __launch_bounds__(256)
attention_mass_kernel(const float* __restrict__ score, const float* __restrict__ ml, float* __restrict__ mass,
                      const int* __restrict__ seq_lens, int N, int Hq, int Hkv, int G) {
    const int h = blockIdx.y, b = blockIdx.z;
    const int t = blockIdx.x * 256 + threadIdx.x;
    const int len = seq_lens ? min(max(seq_lens[b], 0), N) : N;
    if (t >= len) return;
    float acc = 0.f;
    for (int g = 0; g < G; ++g) {
        const long long hq = (long long)b * Hq + h * G + g;
        const float M = ml[hq * 2], L = ml[hq * 2 + 1];
        if (L > 0.f) acc += fast_exp2(score[hq * N + t] - M) / L;
    }
    mass[((long long)b * Hkv + h) * N + t] += acc;
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
// How many clusters of S CTAs of this kernel the device holds at once with `smem` bytes of dynamic shared memory
// (0: that cluster size cannot be launched).  Asked of the driver once per device and size.
template <int D>
static int cluster_room(int device, size_t smem, int S) {
    static int cached[64][MAX_CLUSTER_SPLITS + 1];   // 1 + answer
    static int cached_smem[64] = {0};
    if (device < 0 || device >= 64 || S < 2 || S > MAX_CLUSTER_SPLITS) return 0;
    if (cached_smem[device] != (int)smem) {
        for (int i = 0; i <= MAX_CLUSTER_SPLITS; ++i) cached[device][i] = 0;
        cached_smem[device] = (int)smem;
        if (cudaFuncSetAttribute(gqa_decode_f16_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
            cudaFuncSetAttribute(gqa_decode_f16_kernel<D>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
            cudaGetLastError();
            for (int i = 0; i <= MAX_CLUSTER_SPLITS; ++i) cached[device][i] = 1;   // no cluster launches on this device
        }
    }
    if (cached[device][S] == 0) cached[device][S] = 1 + max_active_clusters(gqa_decode_f16_kernel<D>, dim3(THREADS), smem, S);
    return cached[device][S] - 1;
}

// Short contexts: how many splits per (batch, kv-head) to launch as one cluster, 0 for the ticket combine.  The
// cluster variant replaces the partial sums' trip through global memory (store, fence, ticket, reload by the last CTA)
// by two cluster barriers and loads from the other CTAs' shared memory.  It pays only while every cluster is resident
// at once -- measured on B200: 4 sequences x 8 kv-heads at 4 K tokens 22.5 -> 20.5 us, but 16 sequences at 8 K tokens,
// whose clusters need several waves, 104 -> 135 us (a cluster waits for a whole group of free SMs) -- and clusters
// of 16 of this kernel do not fit eight at a time, so one sequence of 8 kv-heads (16-18 splits) keeps the tickets.
template <int D>
static int cluster_splits(int device, size_t smem, int plan_splits, long long total_tiles, long long pairs) {
    constexpr long long MAX_TILES = 384;   // 24 K tokens: beyond, the fixed cost this removes is a few percent
    if (plan_splits < 2 || total_tiles > MAX_TILES) return 0;
    int S = plan_splits < MAX_CLUSTER_SPLITS ? plan_splits : MAX_CLUSTER_SPLITS;
    const long long tps = (total_tiles + S - 1) / S;
    S = (int)((total_tiles + tps - 1) / tps);
    if (S < 2 || S * 4 < plan_splits * 3) return 0;   // far fewer CTAs than the plan wanted: streaming would cost more than it saves
    return cluster_room<D>(device, smem, S) >= pairs ? S : 0;
}

template <int D>
static int launch_f16(const CUtensorMap& tmK, const CUtensorMap& tmV, const Params& p, int B, cudaStream_t stream) {
    static int configured_smem[64] = {0};
    const size_t smem = Smem<D>::bytes(p.stages);
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && configured_smem[dev] < (int)smem) {
        SKV_CUDA_TRY(cudaFuncSetAttribute(gqa_decode_f16_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured_smem[dev] = (int)smem;
    }
    const dim3 grid = p.list_items > 0 ? dim3(p.Hkv, p.list_items, 1) : dim3(p.Hkv, p.num_splits, B);
    if (p.cluster_combine)
        SKV_CUDA_TRY(launch_pdl_cluster(gqa_decode_f16_kernel<D>, grid, dim3(THREADS), smem, stream, p.num_splits, tmK, tmV, p));
    else
        SKV_CUDA_TRY(launch_pdl(gqa_decode_f16_kernel<D>, grid, dim3(THREADS), smem, stream, tmK, tmV, p));
    SKV_CUDA_TRY(cudaGetLastError());
    return SKV_OK;
}

}  // namespace gqa
}  // namespace skv

using namespace skv;

extern "C" {

// Tuning knobs for experiments: pipeline depth and CTAs resident per SM used
// when the KV length is split.  Values outside the valid range are rejected.
int skv_gqa_set_tuning(int stages, int ctas_per_sm) {
    if (stages < 2 || stages > 6 || ctas_per_sm < 1 || ctas_per_sm > 4)
        return fail(SKV_ERR_BAD_ARG, "tuning out of range: stages=%d ctas_per_sm=%d", stages, ctas_per_sm);
    gqa::tuning().stages = stages;
    gqa::tuning().ctas_per_sm = ctas_per_sm;
    return SKV_OK;
}

// 1 (default): short contexts launch the splits of a (batch, kv-head) as one thread-block cluster and sum them through
// shared memory; 0: always the global-memory partials and ticket.  Results agree to fp32 rounding.  Process-wide.
int skv_gqa_set_cluster_combine(int on) {
    gqa::tuning().cluster_combine = on ? 1 : 0;
    return SKV_OK;
}

// 1: the decode kernels may read K, V, the page table and seq_lens before the previous kernel in the stream has
// completed (valid when that kernel produces none of them, e.g. consecutive layers' decode calls over caches
// written earlier); 0 (default): they wait for it first.  Process-wide.
int skv_gqa_set_early_kv(int on) {
    gqa::tuning().early_kv = on ? 1 : 0;
    return SKV_OK;
}

size_t skv_gqa_decode_workspace_bytes(int B, int N, int Hq, int Hkv, int D, int device) {
    if (B <= 0 || N <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0 || D <= 0) return 0;
    // large enough for either split policy (with or without per-sequence lengths)
    size_t best = 0;
    for (int slots = 1; slots <= 2; ++slots)
        for (int ragged = 0; ragged <= 1; ++ragged) {
            const size_t t = gqa::make_plan(B, N, Hq, Hkv, D, device, ragged != 0, slots).total;
            if (t > best) best = t;
        }
    return best;
}

int skv_gqa_decode_splits(int B, int N, int Hq, int Hkv, int D, int device) {
    if (B <= 0 || N <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0 || D <= 0) return 0;
    return gqa::make_plan(B, N, Hq, Hkv, D, device).splits;
}

// Shared by skv_gqa_decode and skv_gqa_decode_mass; `mass` (optional) adds the attention-mass pass, whose scratch
// (scores [B,Hq,N] and final max/denominator [B,Hq,2], fp32) follows the decode plan in the workspace.
static size_t mass_scratch_bytes(int B, int N, int Hq) {
    return (((size_t)B * Hq * 2 * sizeof(float) + 255) & ~size_t(255)) + (size_t)B * Hq * N * sizeof(float);
}

static int decode_f16_impl(const void* q, const void* k, const void* v, void* out, float* mass, void* workspace,
                           size_t workspace_bytes, int B, int N, int Hq, int Hkv, int D, int kv_dtype,
                           long long kv_stride_b, long long kv_stride_n, long long kv_stride_h, const int* seq_lens,
                           float scale, int device, void* stream) {
    if (!q || !k || !v || !out) return fail(SKV_ERR_BAD_ARG, "skv_gqa_decode: null tensor pointer");
    if (B <= 0 || N <= 0 || Hq <= 0 || Hkv <= 0) return fail(SKV_ERR_BAD_ARG, "skv_gqa_decode: sizes must be positive");
    if (Hq % Hkv != 0) return fail(SKV_ERR_BAD_ARG, "Hq=%d must be divisible by Hkv=%d", Hq, Hkv);
    const int G = Hq / Hkv;
    if (G > gqa::MAX_GROUP) return fail(SKV_ERR_UNSUPPORTED, "group size %d exceeds %d", G, gqa::MAX_GROUP);
    if (D != 128 && D != 64) return fail(SKV_ERR_UNSUPPORTED, "head dim %d not supported (64 or 128)", D);
    if (!(scale > 0.f)) return fail(SKV_ERR_BAD_ARG, "softmax scale must be positive");
    if (kv_dtype != SKV_KV_F16) return fail(SKV_ERR_UNSUPPORTED, "kv_dtype %d not supported by this entry point", kv_dtype);
    if (Hkv > 65535 || B > 65535) return fail(SKV_ERR_UNSUPPORTED, "grid dimension too large");

    DeviceGuard guard(device);
    if (!guard.ok) return fail(SKV_ERR_CUDA, "cannot switch to device %d", device);

    gqa::Plan pl = gqa::make_plan(B, N, Hq, Hkv, D, device, seq_lens != nullptr);
    // the mass scratch sits behind the LARGER of the two split plans, so that its place does not depend on seq_lens
    const size_t plan_max = skv_gqa_decode_workspace_bytes(B, N, Hq, Hkv, D, device);
    const size_t need = mass ? plan_max + mass_scratch_bytes(B, N, Hq) : pl.total;
    if (!workspace || workspace_bytes < need)
        return fail(SKV_ERR_WORKSPACE, "workspace of %zu bytes is smaller than the %zu required", workspace_bytes, need);
    if (reinterpret_cast<uintptr_t>(workspace) & 255) return fail(SKV_ERR_WORKSPACE, "workspace must be 256-byte aligned");

    CUtensorMap tmK, tmV;
    KvMapPos pos, pos2;
    int rc = make_kv_tmap(&tmK, &pos, k, 2, 64, D / 64, B, N, Hkv, kv_stride_b, kv_stride_n, kv_stride_h, gqa::TILE);
    if (rc) return rc;
    rc = make_kv_tmap(&tmV, &pos2, v, 2, 64, D / 64, B, N, Hkv, kv_stride_b, kv_stride_n, kv_stride_h, gqa::TILE);
    if (rc) return rc;

    gqa::Params p;
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    p.q = static_cast<const __half*>(q);
    p.out = static_cast<__half*>(out);
    p.tickets = reinterpret_cast<int*>(ws + pl.off_tickets);
    p.status = reinterpret_cast<int*>(ws + pl.off_status);
    p.partial_ml = reinterpret_cast<float*>(ws + pl.off_ml);
    p.partial_o = reinterpret_cast<float*>(ws + pl.off_o);
    p.seq_lens = seq_lens;
    p.N = N; p.Hq = Hq; p.Hkv = Hkv; p.G = G;
    p.tiles_per_split = pl.tiles_per_split;
    p.num_splits = pl.splits;
    p.stages = gqa::tuning().stages;
    p.early_kv = gqa::tuning().early_kv;
    {   // ragged lengths, few pairs: one wave of CTAs from a device-side work list (the condition of the 8-bit kernel)
        const int slots_total = sm_count(device) * gqa::tuning().ctas_per_sm;
        const int waves = gqa::tuning().ragged_worklist;
        const bool worklist = seq_lens != nullptr && waves > 0 && B <= 64 && (long long)B * Hkv * 8 <= slots_total;
        p.list_items = worklist ? slots_total * waves / Hkv : 0;
        p.B = B;
    }
    p.cluster_combine = 0;
    if (gqa::tuning().cluster_combine && !mass && p.list_items == 0) {
        const long long total_tiles = (N + gqa::TILE - 1) / gqa::TILE;
        const size_t smem = D == 128 ? gqa::Smem<128>::bytes(p.stages) : gqa::Smem<64>::bytes(p.stages);
        const int S = D == 128 ? gqa::cluster_splits<128>(device, smem, pl.splits, total_tiles, (long long)B * Hkv)
                               : gqa::cluster_splits<64>(device, smem, pl.splits, total_tiles, (long long)B * Hkv);
        if (S > 0) {
            p.cluster_combine = 1;
            p.num_splits = S;
            p.tiles_per_split = (int)((total_tiles + S - 1) / S);
        }
    }
    p.q_stride_b = (long long)Hq * D; p.q_stride_h = D;
    p.o_stride_b = (long long)Hq * D; p.o_stride_h = D;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.pos = pos;
    p.ml_final = mass ? reinterpret_cast<float*>(ws + plan_max) : nullptr;
    p.score_out = mass ? reinterpret_cast<float*>(ws + plan_max + (((size_t)B * Hq * 2 * sizeof(float) + 255) & ~size_t(255))) : nullptr;

    cudaStream_t st = static_cast<cudaStream_t>(stream);
    rc = D == 128 ? gqa::launch_f16<128>(tmK, tmV, p, B, st) : gqa::launch_f16<64>(tmK, tmV, p, B, st);
    if (rc || !mass) return rc;
    dim3 grid((N + 255) / 256, Hkv, B);
    gqa::attention_mass_kernel<<<grid, 256, 0, st>>>(p.score_out, p.ml_final, mass, seq_lens, N, Hq, Hkv, G);
    SKV_CUDA_TRY(cudaGetLastError());
    return SKV_OK;
}

int skv_gqa_decode(const void* q, const void* k, const void* v, void* out, void* workspace, size_t workspace_bytes,
                   int B, int N, int Hq, int Hkv, int D, int kv_dtype, const float* k_scale, const float* v_scale,
                   long long kv_stride_b, long long kv_stride_n, long long kv_stride_h, const int* seq_lens,
                   float scale, int device, void* stream) {
    (void)k_scale; (void)v_scale;
    return decode_f16_impl(q, k, v, out, nullptr, workspace, workspace_bytes, B, N, Hq, Hkv, D, kv_dtype, kv_stride_b,
                           kv_stride_n, kv_stride_h, seq_lens, scale, device, stream);
}

// Dense decode that also accumulates every cached token's attention mass (summed over the query heads of its
// kv-head) into `mass` fp32 [B, Hkv, N]: the importance scores an eviction policy feeds to skv_kv_evict_quant.
size_t skv_gqa_decode_mass_workspace_bytes(int B, int N, int Hq, int Hkv, int D, int device) {
    const size_t base = skv_gqa_decode_workspace_bytes(B, N, Hq, Hkv, D, device);
    return base ? base + mass_scratch_bytes(B, N, Hq) : 0;
}

int skv_gqa_decode_mass(const void* q, const void* k, const void* v, void* out, float* mass, void* workspace,
                        size_t workspace_bytes, int B, int N, int Hq, int Hkv, int D, long long kv_stride_b,
                        long long kv_stride_n, long long kv_stride_h, const int* seq_lens, float scale, int device,
                        void* stream) {
    if (!mass) return fail(SKV_ERR_BAD_ARG, "skv_gqa_decode_mass: null mass pointer");
    return decode_f16_impl(q, k, v, out, mass, workspace, workspace_bytes, B, N, Hq, Hkv, D, SKV_KV_F16, kv_stride_b,
                           kv_stride_n, kv_stride_h, seq_lens, scale, device, stream);
}

#ifdef SKV_PROFILE_PHASES
int skv_debug_phase_ts_f16(unsigned long long* out) {
    return cudaMemcpyFromSymbol(out, skv_phase_ts, sizeof(unsigned long long) * 32) == cudaSuccess ? 0 : -4;
}
#endif

// ---------------------------------------------------------------------------
// Allocation-free variant of skv_gqa_decode.
//
// Some callers have no device allocator to take a workspace from: a serving
// process that gave all remaining HBM to its KV page pool at start-up (a later
// cudaMalloc fails, or stalls every stream while the driver looks for memory),
// or a plain C / Go host that links this library without torch and its caching
// allocator.  For them the split-KV scratch (status word, tickets, fp32
// partials) lives in a fixed array inside the library image instead.
//
//   * The array is SKV_GQA_STATIC_SCRATCH_BYTES (4 MiB) per GPU that loads the
//     library, held until the process exits.  A problem whose
//     skv_gqa_decode_workspace_bytes() exceeds that is rejected with
//     SKV_ERR_WORKSPACE; use skv_gqa_decode with a caller workspace then.
//   * In host code the array's name is only a handle: its device address is
//     looked up once per device with cudaGetSymbolAddress (device made current
//     first) and that pointer is what the kernel receives.  The lookup happens
//     in the FIRST call on each device, which therefore should be made before
//     any stream capture begins on that device.
//   * All calls on one GPU share the array and it keeps the previous call's
//     contents: the part that must start at zero (status word and tickets) is
//     cleared on `stream` before every launch.  Two calls that can overlap on
//     the same GPU (different streams, no ordering) race on it -- serialise
//     them, or use skv_gqa_decode with separate workspaces.
//   * Nothing here calls cudaMalloc, cudaFree or any allocating library routine.
// ---------------------------------------------------------------------------
#define SKV_GQA_STATIC_SCRATCH_BYTES (4u << 20)
static_assert(SKV_GQA_STATIC_SCRATCH_BYTES == 4194304u, "keep in step with include/skv_b200.h");

static __device__ __align__(256) unsigned char skv_gqa_static_scratch[SKV_GQA_STATIC_SCRATCH_BYTES];
static void* g_static_scratch_ptr[64] = {nullptr};  // device address of the array, per device ordinal
static std::mutex g_static_scratch_mu;

// Device address of the array on `device` (which must be current).  The one-time lookup refuses to run while `stream`
// is being captured: a capture must not be the first thing that touches the array on a device.
static int static_scratch_address(int device, cudaStream_t stream, void** out) {
    std::lock_guard<std::mutex> lock(g_static_scratch_mu);
    void* scratch = g_static_scratch_ptr[device];
    if (!scratch) {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(stream, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone)
            return fail(SKV_ERR_CUDA, "the first skv_gqa_decode_noalloc call on a device must be made outside stream capture");
        cudaError_t e = cudaGetSymbolAddress(&scratch, skv_gqa_static_scratch);
        if (e != cudaSuccess || !scratch)
            return fail(SKV_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed: %s", cudaGetErrorString(e));
        g_static_scratch_ptr[device] = scratch;
    }
    *out = scratch;
    return SKV_OK;
}

int skv_gqa_decode_noalloc(const void* q, const void* k, const void* v, void* out, int B, int N, int Hq, int Hkv,
                           int D, long long kv_stride_b, long long kv_stride_n, long long kv_stride_h,
                           const int* seq_lens, float scale, int device, void* stream) {
    if (B <= 0 || N <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || Hq % Hkv != 0)
        return fail(SKV_ERR_BAD_ARG, "skv_gqa_decode_noalloc: sizes must be positive and Hq divisible by Hkv");
    if (device < 0 || device >= 64) return fail(SKV_ERR_BAD_ARG, "device ordinal %d out of range", device);
    DeviceGuard guard(device);
    if (!guard.ok) return fail(SKV_ERR_CUDA, "cannot switch to device %d", device);

    const gqa::Plan pl = gqa::make_plan(B, N, Hq, Hkv, D, device, seq_lens != nullptr);
    if (pl.total > (size_t)SKV_GQA_STATIC_SCRATCH_BYTES)
        return fail(SKV_ERR_WORKSPACE,
                    "this problem needs %zu bytes of scratch but the built-in array holds %u: "
                    "call skv_gqa_decode with a caller-provided workspace",
                    pl.total, (unsigned)SKV_GQA_STATIC_SCRATCH_BYTES);
    void* scratch = nullptr;
    const int rc = static_scratch_address(device, static_cast<cudaStream_t>(stream), &scratch);
    if (rc) return rc;
    // The tickets must be zero when the kernel starts; the partials need no clearing.  The status word in front of
    // them is NOT cleared: a bounded wait that ran out stays visible to skv_gqa_decode_noalloc_status.
    SKV_CUDA_TRY(cudaMemsetAsync(static_cast<unsigned char*>(scratch) + pl.off_tickets, 0, pl.off_ml - pl.off_tickets,
                                 static_cast<cudaStream_t>(stream)));
    return skv_gqa_decode(q, k, v, out, scratch, (size_t)SKV_GQA_STATIC_SCRATCH_BYTES, B, N, Hq, Hkv, D, SKV_KV_F16,
                          nullptr, nullptr, kv_stride_b, kv_stride_n, kv_stride_h, seq_lens, scale, device, stream);
}

// The status word of the built-in scratch array on `device` (bit SKV_DEV_TIMEOUT: a bounded wait inside the kernel
// gave up); the word keeps its bits until the process ends.  Synchronises `stream`.  Allocates nothing.
int skv_gqa_decode_noalloc_status(int device, void* stream, int* status_out) {
    if (!status_out) return fail(SKV_ERR_BAD_ARG, "skv_gqa_decode_noalloc_status: null pointer");
    if (device < 0 || device >= 64) return fail(SKV_ERR_BAD_ARG, "device ordinal %d out of range", device);
    DeviceGuard guard(device);
    if (!guard.ok) return fail(SKV_ERR_CUDA, "cannot switch to device %d", device);
    void* scratch = nullptr;
    const int rc = static_scratch_address(device, static_cast<cudaStream_t>(stream), &scratch);
    if (rc) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    SKV_CUDA_TRY(cudaMemcpyAsync(status_out, scratch, sizeof(int), cudaMemcpyDeviceToHost, st));
    SKV_CUDA_TRY(cudaStreamSynchronize(st));
    return SKV_OK;
}

}  // extern "C"
