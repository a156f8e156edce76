// Token-sparse decode attention: score every cached key, keep the top_k best
// (plus the first sink_tokens positions), softmax over the kept scores only and
// sum the kept value rows.
//
// Replaces sparse_kv_attn_kernel / kv_evict_quant_forward of the reference
// (csrc/kernels/kv_evict_quant.cu:107-269, :272-364) and follows the arithmetic of
// its PyTorch path _reference_sparse_attention (sparse_kv/attention.py:25-38),
// including the sink prefix, which the reference's CUDA path silently ignores, and
// with an exact top-k instead of the reference kernel's lossy per-thread heaps.
//
// Two launches:
//   1. token_scores_mma_kernel (decode shape, D = 64 / 128: K by TMA through a ring, scores on the
//      tensor cores) or token_scores_kernel (16-byte loads, one row of D channels per D/8 lanes)
//      -- streams K once (HBM-bound), scores to an fp32 scratch [rows, T]; for long rows every
//      CTA also leaves the top-k of its chunk as candidates;
//   2. token_select_attend_kernel -- one 1024-thread CTA per (b, h, query): exact top-k over the
//      candidates or the scratch (L2 resident; skv_select.cuh), softmax, gather of the kept V rows.
#include "skv_common.cuh"
#include "skv_select.cuh"
#include "skv_tmap.cuh"

namespace skv {
namespace tsp {

constexpr int SCORE_THREADS = 256;
constexpr int ATT_THREADS = 1024;
constexpr int MAX_KEEP = 4096;  // top_k + sink_tokens upper bound
constexpr int MAX_CAND_K = 256;  // largest top_k served by the per-chunk candidate path

// Chunk slots reserved in the workspace for candidates (scores CTAs: about 8 per SM plus one per row).
inline long long cand_capacity_chunks(long long rows) { return 4096 + 2 * rows; }

struct ScoreParams {
    const __half* q;   // element (b,h,s,d) at b*q_sb + h*q_sh + s*q_ss + d
    const __half* k;   // element (b,h,t,d) at b*k_sb + h*k_sh + t*k_st + d
    float* scores;     // [B, H, S, T]
    int H, S, T;
    long long q_sb, q_sh, q_ss, k_sb, k_sh, k_st;
    float scale;
    // candidate mode (cand_k > 0): every CTA also leaves the cand_k best tokens of its chunk
    float* cand_score;   // [rows, nchunks, cand_k], -inf padded
    int* cand_pos;       // [rows, nchunks, cand_k], -1 padded
    int cand_k;
};

// Rows shorter than this skip the per-chunk candidates: the row-wide select over all scores is cheaper there.
#ifndef SKV_CAND_MIN_T
#define SKV_CAND_MIN_T 32768
#endif

// grid (ceil(T / tokens_per_cta), H, B*S)
template <int D>
__global__ void __launch_bounds__(SCORE_THREADS)
token_scores_kernel(const ScoreParams p, int tokens_per_cta) {
    pdl_launch_dependents();  // the kernel that consumes these results may be scheduled now; it waits for this grid to finish
    constexpr int LPR = D / 8;      // lanes per key row
    constexpr int RPW = 32 / LPR;   // rows per warp-wide load
    constexpr int SUB = 32 / RPW;   // loads per 32 tokens
    __shared__ float stage[SCORE_THREADS / 32][32];
    extern __shared__ uint32_t cand_sm[];  // candidate mode: chunk scores [tokens_per_cta], select scratch, positions
    float* chunk_sc = reinterpret_cast<float*>(cand_sm);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane % LPR, rw = lane / LPR;
    const int h = blockIdx.y, b = blockIdx.z / p.S, s = blockIdx.z % p.S;

    float q[8];
    {
        const uint4 qv = *reinterpret_cast<const uint4*>(p.q + b * p.q_sb + h * p.q_sh + s * p.q_ss + sub * 8);
        const __half2* hq = reinterpret_cast<const __half2*>(&qv);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(hq[i]);
            q[2 * i] = f.x;
            q[2 * i + 1] = f.y;
        }
    }
    const __half* kbase = p.k + b * p.k_sb + h * p.k_sh + sub * 8;
    float* srow = p.scores + (((long long)b * p.H + h) * p.S + s) * p.T;
    const int t0 = blockIdx.x * tokens_per_cta, t1 = min(p.T, t0 + tokens_per_cta);

    for (int base = t0 + warp * 32; base < t1; base += (SCORE_THREADS / 32) * 32) {
        uint4 kv[SUB];
#pragma unroll
        for (int j = 0; j < SUB; ++j) {
            // rows past the end are clamped to the last row (their scores are never stored): loads without a
            // condition are all issued before the first use
            const int t = min(base + j * RPW + rw, t1 - 1);
            kv[j] = ld_stream16(kbase + (long long)t * p.k_st);
        }
#pragma unroll
        for (int j = 0; j < SUB; ++j) {
            float d = dot8(kv[j], q);
#pragma unroll
            for (int o = LPR / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
            if (sub == 0) stage[warp][j * RPW + rw] = d * p.scale;
        }
        __syncwarp();
        if (base + lane < t1) {
            srow[base + lane] = stage[warp][lane];
            if (p.cand_k > 0) chunk_sc[base + lane - t0] = stage[warp][lane];
        }
        __syncwarp();
    }
    if (p.cand_k > 0) {
        // The global top-k is a subset of the union of every chunk's top-k, so the row-wide selection later
        // only has to look at nchunks * cand_k candidates instead of all T scores.
        uint32_t* tk = cand_sm + tokens_per_cta;
        int* csel = reinterpret_cast<int*>(tk + TopkSmem<SCORE_THREADS>::WORDS);
        const int n = t1 - t0, kc = min(p.cand_k, n);
        __syncthreads();
        block_topk_fast<SCORE_THREADS, 16>(chunk_sc, n, kc, csel, tk);
        __syncthreads();
        const long long row = ((long long)b * p.H + h) * p.S + s;
        const long long o = (row * gridDim.x + blockIdx.x) * p.cand_k;
        for (int i = threadIdx.x; i < p.cand_k; i += SCORE_THREADS) {
            p.cand_pos[o + i] = i < kc ? t0 + csel[i] : -1;
            p.cand_score[o + i] = i < kc ? chunk_sc[csel[i]] : -INFINITY;
        }
    }
}

// Tensor-core variant of the scoring kernel for one query per (b, h) (decode) and D = 64 or 128.  The register-load
// kernel above spends about 40 instructions per KB of keys on conversions, FMAs and lane reductions and reaches 0.73 of
// the copy bandwidth; here the keys stream like K in the dense decode kernel -- TMA boxes of 128 tokens x 64 channels
// (128-byte swizzle, evict-first) into a 2- or 3-stage ring -- and a tile's scores are one [128 tokens x D] . [D x 8] product
// (ldmatrix + mma.sync.m16n8k16, tokens on the M side, the query in column 0 of the N side).  Same grid, chunks and
// per-chunk candidates as the kernel above.  Thread 0 refills a stage right after the block-wide barrier that ends
// its previous use; every wait is bounded, and a wait that runs out sets SKV_DEV_TIMEOUT and ends the CTA's loop.
// grid (ceil(T / tokens_per_cta), H, B)
constexpr int MMA_TILE = 128;     // tokens per stage: 16 per warp
// Staggered chunks: chunk x of n covers the tiles [chunk_first_tile(x), chunk_first_tile(x + 1)) of a row of nt tiles,
// with lengths falling linearly from 1.5 to 0.5 times the mean.  CTAs of equal chunks start together, stream together
// and run their candidate selection together, wave after wave, and the memory system idles during every selection;
// unequal chunks spread the selections over time.
__host__ __device__ inline int chunk_first_tile(int x, int n, int nt) {
    return (int)((long long)nt * (3LL * x * n - (long long)x * x) / (2LL * n * n));
}
template <int D>
__host__ __device__ constexpr int mma_stage_bytes() { return MMA_TILE * D * 2; }
template <int D, int MMA_STAGES>
__host__ __device__ constexpr size_t mma_ring_bytes() { return (size_t)MMA_STAGES * mma_stage_bytes<D>() + 64; }

// MMA_STAGES = 2 with three CTAs per SM for chunks of up to 2 K tokens (the per-chunk candidate selection of one CTA
// then overlaps two others' streaming), 3 with two CTAs per SM for longer chunks; the host takes the long ring and
// chunks of up to 3.5 K tokens from 64K x 32 rows up (measured: 64K 103 against 107 us, 128K 189 against 196 us with
// the short ring).
template <int D, int MMA_STAGES>
__global__ void __launch_bounds__(SCORE_THREADS, MMA_STAGES == 2 ? 3 : 2)
token_scores_mma_kernel(const __grid_constant__ CUtensorMap tmK, const ScoreParams p, const KvMapPos pos,
                        int tokens_per_cta, int stagger_tiles, int* status) {
    pdl_launch_dependents();
    SKV_PHASE(0);
    constexpr int NH = D / 64, KSTEPS = D / 16, HALF_BYTES = MMA_TILE * 128, STAGE = mma_stage_bytes<D>();
    extern __shared__ uint8_t mma_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(mma_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t ring = smem_u32(smem);
    const uint32_t full_bar = ring + MMA_STAGES * STAGE;
    float* chunk_sc = reinterpret_cast<float*>(smem + mma_ring_bytes<D, MMA_STAGES>());   // candidate mode: [tokens_per_cta]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, tq = lane & 3, lj = lane >> 3, r8 = lane & 7;
    const int h = blockIdx.y, b = blockIdx.z;
    // stagger_tiles > 0: the row's tile count; the chunks are the staggered ones
    const int t0 = stagger_tiles > 0 ? chunk_first_tile(blockIdx.x, gridDim.x, stagger_tiles) * MMA_TILE : blockIdx.x * tokens_per_cta;
    const int t1 = stagger_tiles > 0 ? min(p.T, chunk_first_tile(blockIdx.x + 1, gridDim.x, stagger_tiles) * MMA_TILE)
                                     : min(p.T, t0 + tokens_per_cta);
    const int ntiles = (t1 - t0 + MMA_TILE - 1) / MMA_TILE;
    if (tid == 0) {
        for (int s = 0; s < MMA_STAGES; ++s) mbar_init(full_bar + s * 8, 1);
        fence_barrier_init();
    }
    __syncthreads();
    const uint64_t policy = l2_policy_evict_first();
    auto issue = [&](int tile) {   // thread 0 only
        const int s = tile % MMA_STAGES;
        const uint32_t bar = full_bar + s * 8, dst = ring + s * STAGE;
        mbar_expect_tx(bar, STAGE);
#pragma unroll
        for (int hf = 0; hf < NH; ++hf) {
            int c[5] = {0, 0, 0, 0, 0};
#pragma unroll
            for (int i = 1; i < 5; ++i) c[i] = (i == pos.half) ? hf : (i == pos.tok) ? t0 + tile * MMA_TILE : (i == pos.head) ? h : b;
            tma_load_5d(dst + hf * HALF_BYTES, &tmK, bar, c[0], c[1], c[2], c[3], c[4], policy);
        }
    };
    if (tid == 0) {
        tma_prefetch_desc(&tmK);
        for (int i = 0; i < MMA_STAGES - 1 && i < ntiles; ++i) issue(i);
    }
    // the query as the B operand: column 0 of the 8-wide N side, the other columns zero
    uint32_t qb[KSTEPS][2];
    {
        const __half* qrow = p.q + b * p.q_sb + h * p.q_sh;
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {
            qb[kk][0] = g == 0 ? *reinterpret_cast<const uint32_t*>(qrow + kk * 16 + tq * 2) : 0u;
            qb[kk][1] = g == 0 ? *reinterpret_cast<const uint32_t*>(qrow + kk * 16 + 8 + tq * 2) : 0u;
        }
    }
    float* srow = p.scores + ((long long)b * p.H + h) * p.T;
    const uint32_t a_row_off = (uint32_t)((warp * 16 + (lj & 1) * 8 + r8) * 128);   // this lane's ldmatrix row (row & 7 == r8)
    for (int i = 0; i < ntiles; ++i) {
        // (everybody has passed the barrier that ended tile i-1, so the stage tile i + STAGES - 1 goes into is free)
        if (tid == 0 && i + MMA_STAGES - 1 < ntiles) issue(i + MMA_STAGES - 1);
        const int s = i % MMA_STAGES;
        int ok = mbar_wait(full_bar + s * 8, (uint32_t)((i / MMA_STAGES) & 1)) ? 1 : 0;
        if (ok) {
            const uint32_t base = ring + s * STAGE + a_row_off;
            float acc0[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int kk = 0; kk < KSTEPS; ++kk) {
                const int c = 2 * kk + (lj >> 1);
                uint32_t a[4];
                ldsm_x4(base + (uint32_t)(c >> 3) * HALF_BYTES + (uint32_t)(((c & 7) ^ r8) << 4), a[0], a[1], a[2], a[3]);
                if (kk & 1) mma_f16(acc1, a, qb[kk][0], qb[kk][1]);
                else mma_f16(acc0, a, qb[kk][0], qb[kk][1]);
            }
            if (tq == 0) {   // column 0: the query; rows g and g + 8 of this warp's 16 tokens
                const int tok = t0 + i * MMA_TILE + warp * 16 + g;
                const float v0 = (acc0[0] + acc1[0]) * p.scale, v1 = (acc0[2] + acc1[2]) * p.scale;
                if (tok < t1) {
                    srow[tok] = v0;
                    if (p.cand_k > 0) chunk_sc[tok - t0] = v0;
                }
                if (tok + 8 < t1) {
                    srow[tok + 8] = v1;
                    if (p.cand_k > 0) chunk_sc[tok + 8 - t0] = v1;
                }
            }
        }
        if (!__syncthreads_and(ok)) {   // also: everybody is done with tile i
            if (tid == 0) {
                atomicOr(status, SKV_DEV_TIMEOUT);
                // copies already issued for later tiles still target this CTA's shared memory: give them a (bounded)
                // chance to land before the CTA may leave
                for (int t = i + 1; t < ntiles && t < i + MMA_STAGES; ++t)
                    mbar_wait(full_bar + (t % MMA_STAGES) * 8, (uint32_t)((t / MMA_STAGES) & 1));
            }
            __syncthreads();
            break;
        }
    }
    SKV_PHASE(1);
    if (p.cand_k > 0) {   // as in token_scores_kernel; the select scratch reuses the drained ring (every copy has landed)
        uint32_t* tk = reinterpret_cast<uint32_t*>(smem);
        int* csel = reinterpret_cast<int*>(tk + TopkSmem<SCORE_THREADS>::WORDS);
        const int n = t1 - t0, kc = min(p.cand_k, n);
        __syncthreads();
        block_topk_fast<SCORE_THREADS, 16>(chunk_sc, n, kc, csel, tk);
        __syncthreads();
        const long long row = (long long)b * p.H + h;
        const long long o = (row * gridDim.x + blockIdx.x) * p.cand_k;
        for (int i = tid; i < p.cand_k; i += SCORE_THREADS) {
            p.cand_pos[o + i] = i < kc ? t0 + csel[i] : -1;
            p.cand_score[o + i] = i < kc ? chunk_sc[csel[i]] : -INFINITY;
        }
    }
    SKV_PHASE(2);
}

struct AttendParams {
    const float* scores;  // [rows, T]
    const __half* v;      // element (b,h,t,d) at b*v_sb + h*v_sh + t*v_st + d
    __half* out;          // [rows, D]
    int* topk_idx;        // optional [rows, top_k], ascending, -1 padded
    int H, S, T, top_k, sink;
    long long v_sb, v_sh, v_st;
    const float* cand_score;  // candidate mode: [rows, nc]; null otherwise
    const int* cand_pos;
    int nc;
};

// grid (rows = B*H*S)
template <int D>
__global__ void __launch_bounds__(ATT_THREADS)
token_select_attend_kernel(const AttendParams p) {
    SKV_PHASE(3);
    pdl_wait_prior_grids();   // launched as a programmatic dependent of the scoring kernel: its results are complete from here on
    SKV_PHASE(4);
    constexpr int LPR = D / 8;
    constexpr int GROUPS = ATT_THREADS / LPR;  // value rows gathered in parallel
    extern __shared__ uint32_t dsm[];
    uint32_t* tk = dsm;                                             // TopkSmem words
    int* sel = reinterpret_cast<int*>(tk + TopkSmem<ATT_THREADS>::WORDS);  // [MAX_KEEP]
    float* w = reinterpret_cast<float*>(sel + MAX_KEEP);            // [MAX_KEEP]
    float* red = w + MAX_KEEP;                                      // [GROUPS][D] (aliases nothing above)
    __shared__ float bcast[2];

    const int row = blockIdx.x;
    const int s_ = row % p.S, h = (row / p.S) % p.H, b = row / (p.S * p.H);
    (void)s_;
    const float* sc = p.scores + (long long)row * p.T;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kk = min(p.top_k, p.T), sink = min(max(p.sink, 0), p.T);

    // the scores of the sink prefix are needed whatever gets selected: on their way before the selection starts
    const float sink_sc0 = tid < sink ? sc[tid] : 0.f;
    // 1. exact top-k, ascending positions, into sel[sink ...)
    int* top = sel + sink;
    float* top_sc = w + sink;   // candidate mode: the kept candidates' scores travel with their positions
    if (p.cand_score) {
        // candidates are ordered by token position (chunk by chunk, ascending inside a chunk), so "equal scores:
        // lower candidate index first" is the same rule as "lower token position first"
        block_topk_fast<ATT_THREADS, 4>(p.cand_score + (long long)row * p.nc, p.nc, kk, top, tk);
        __syncthreads();
        for (int i = tid; i < kk; i += ATT_THREADS) {
            const long long ci = (long long)row * p.nc + SKV_INDEX(top[i], p.nc);
            top[i] = p.cand_pos[ci];
            top_sc[i] = p.cand_score[ci];   // the same number the scoring kernel stored at scores[position]
        }
        __syncthreads();
    } else {
        block_topk_fast<ATT_THREADS, 8>(sc, p.T, kk, top, tk);
    }
    SKV_PHASE(5);
    if (p.topk_idx) {
        for (int i = tid; i < p.top_k; i += ATT_THREADS) p.topk_idx[(long long)row * p.top_k + i] = i < kk ? top[i] : -1;
    }
    __syncthreads();
    const int grp = tid / LPR, sub = tid % LPR;
    const __half* vbase = p.v + b * p.v_sb + h * p.v_sh + sub * 8;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    float inv;
    if (sink + kk <= 64) {
        // Few kept tokens (the usual decode case): every warp works the kept set out for itself -- lane l holds the
        // weights of kept tokens l and l + 32 and hands them out by shuffle -- so that nothing is compacted in shared
        // memory and no block-wide barrier stands between the selection and the gather.
        const int tp0 = lane < kk ? top[lane] : 0x7fffffff, tp1 = lane + 32 < kk ? top[lane + 32] : 0x7fffffff;
        const int c = __popc(__ballot_sync(0xffffffffu, tp0 < sink)) + __popc(__ballot_sync(0xffffffffu, tp1 < sink));
        const int n = sink + kk - c;   // kept token j: position j for j < sink, top[c + j - sink] after that
        constexpr int PASSES = (64 + GROUPS - 1) / GROUPS;   // value rows per thread
        uint4 vv[PASSES];
#pragma unroll
        for (int u = 0; u < PASSES; ++u) {   // (rows past the kept set: a clamped row, weighted zero below)
            const int j = min(u * GROUPS + grp, n - 1);
            const int pos = j < sink ? j : top[c + j - sink];
            vv[u] = *reinterpret_cast<const uint4*>(vbase + (long long)SKV_INDEX(pos, p.T) * p.v_st);
        }
        float x[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int j = lane + 32 * r;
            x[r] = -INFINITY;
            if (j < n) x[r] = j < sink ? sc[j] : (p.cand_score ? top_sc[c + j - sink] : sc[SKV_INDEX(top[c + j - sink], p.T)]);
        }
        const float mxw = warp_max(fmaxf(x[0], x[1]));
        const float e0 = lane < n ? __expf(x[0] - mxw) : 0.f, e1 = lane + 32 < n ? __expf(x[1] - mxw) : 0.f;
        inv = 1.f / warp_sum(e0 + e1);
        SKV_PHASE(7);
#pragma unroll
        for (int u = 0; u < PASSES; ++u) {
            const int j = u * GROUPS + grp;
            const float w0 = __shfl_sync(0xffffffffu, e0, j & 31), w1 = __shfl_sync(0xffffffffu, e1, j & 31);
            const float wj = j < n ? ((j & 32) ? w1 : w0) : 0.f;
            const __half2* hv = reinterpret_cast<const __half2*>(&vv[u]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __half22float2(hv[i]);
                acc[2 * i] = fmaf(wj, f.x, acc[2 * i]);
                acc[2 * i + 1] = fmaf(wj, f.y, acc[2 * i + 1]);
            }
        }
    } else {
        // 2. kept set = sink prefix U {top positions >= sink}: drop the leading top entries that fall inside the prefix
        int c = 0;  // top is ascending, so entries < sink form a prefix of length c
        {
            int lo = 0, hi = kk;
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (top[mid] < sink) lo = mid + 1; else hi = mid;
            }
            c = lo;
        }
        const int n = sink + kk - c;
        __syncthreads();
        // compact in place: positions [0, sink) then top[c ..)
        for (int base = 0; base < kk - c; base += ATT_THREADS) {
            const int i = base + tid;
            const int v = i < kk - c ? top[c + i] : 0;
            const float vs = (p.cand_score && i < kk - c) ? top_sc[c + i] : 0.f;
            __syncthreads();
            if (i < kk - c) {
                sel[sink + i] = v;
                if (p.cand_score) w[sink + i] = vs;
            }
        }
        for (int i = tid; i < sink; i += ATT_THREADS) sel[i] = i;
        __syncthreads();

        // the first pass of value rows: their addresses are known now, their weights only after the softmax
        uint4 v_first = make_uint4(0u, 0u, 0u, 0u);
        if (grp < n) v_first = *reinterpret_cast<const uint4*>(vbase + (long long)SKV_INDEX(sel[grp], p.T) * p.v_st);

        SKV_PHASE(6);
        // 3. softmax over the kept scores
        float mx = -INFINITY;
        for (int i = tid; i < n; i += ATT_THREADS) {
            const float x = i < sink ? (i == tid ? sink_sc0 : sc[i]) : (p.cand_score ? w[i] : sc[SKV_INDEX(sel[i], p.T)]);
            w[i] = x;
            mx = fmaxf(mx, x);
        }
        mx = warp_max(mx);
        if (lane == 0) red[warp] = mx;
        __syncthreads();
        if (warp == 0) {
            float m2 = lane < ATT_THREADS / 32 ? red[lane] : -INFINITY;
            m2 = warp_max(m2);
            if (lane == 0) bcast[0] = m2;
        }
        __syncthreads();
        mx = bcast[0];
        float sum = 0.f;
        for (int i = tid; i < n; i += ATT_THREADS) {
            const float e = __expf(w[i] - mx);
            w[i] = e;
            sum += e;
        }
        sum = warp_sum(sum);
        __syncthreads();
        if (lane == 0) red[warp] = sum;
        __syncthreads();
        if (warp == 0) {
            float s2 = lane < ATT_THREADS / 32 ? red[lane] : 0.f;
            s2 = warp_sum(s2);
            if (lane == 0) bcast[1] = s2;
        }
        __syncthreads();
        inv = 1.f / bcast[1];

        SKV_PHASE(7);
        // 4. out = sum_j w_j V[sel_j] / sum
        for (int j = grp; j < n; j += GROUPS) {
            const uint4 vv = j == grp ? v_first : *reinterpret_cast<const uint4*>(vbase + (long long)SKV_INDEX(sel[j], p.T) * p.v_st);
            const float wj = w[j];
            const __half2* hv = reinterpret_cast<const __half2*>(&vv);
    #pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __half22float2(hv[i]);
                acc[2 * i] = fmaf(wj, f.x, acc[2 * i]);
                acc[2 * i + 1] = fmaf(wj, f.y, acc[2 * i + 1]);
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 8; ++i) red[grp * D + sub * 8 + i] = acc[i];
    __syncthreads();
    for (int d = tid; d < D; d += ATT_THREADS) {
        float o = 0.f;
#pragma unroll 8
        for (int g2 = 0; g2 < GROUPS; ++g2) o += red[g2 * D + d];
        p.out[(long long)row * D + d] = __float2half_rn(o * inv);
    }
    SKV_PHASE(8);
}

template <int D>
static size_t attend_smem() {
    return (size_t)TopkSmem<ATT_THREADS>::WORDS * 4 + (size_t)MAX_KEEP * 8 + (size_t)(ATT_THREADS / (D / 8)) * D * 4;
}

// 1 (default): one query per (b, h) with D = 64 or 128 is scored by the tensor-core kernel; 0: always the register-load
// kernel.  The two sum the same exact products in different orders.
inline int& mma_scores_flag() { static int on = 1; return on; }
inline int& stagger_flag() { static int on = 1; return on; }   // chunks of unequal length for the tensor-core scoring kernel

template <int D>
static int launch(const ScoreParams& sp, const AttendParams& ap, int B, int device, cudaStream_t st, float* cand_base, int* status) {
    static bool configured[64] = {false};
    const size_t smem = attend_smem<D>();
    if (device < 64 && !configured[device]) {
        SKV_CUDA_TRY(cudaFuncSetAttribute(token_select_attend_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured[device] = true;
    }
    // enough CTAs to fill the machine a few times over, at least 512 tokens each
    const long long rows = (long long)B * sp.H * sp.S;
#ifndef SKV_TOKEN_CTAS_PER_SM
#define SKV_TOKEN_CTAS_PER_SM 8
#endif
    long long want = ((long long)sm_count(device) * SKV_TOKEN_CTAS_PER_SM + rows - 1) / rows;
    int tokens_per_cta = (int)((sp.T + want - 1) / want);
    tokens_per_cta = ((tokens_per_cta + 255) / 256) * 256;
    if (tokens_per_cta < 512) tokens_per_cta = 512;
    const bool mma_path = (D == 64 || D == 128) && mma_scores_flag() && sp.S == 1;
    dim3 g1((sp.T + tokens_per_cta - 1) / tokens_per_cta, sp.H, B * sp.S);
    // Staggered chunks for the tensor-core kernel: as many as keep the longest (the first) within the tokens that the
    // ring's shared-memory budget leaves for a chunk's scores (2048 beside the short ring, 3584 beside the long one).
    int stagger_tiles = 0;
    const int stagger_cap = tokens_per_cta <= 1536 ? 2048 : 3584;   // (64K x 32 rows: 27 long chunks beside the long ring 103 us, 48 short ones 107 us)
    if (mma_path && stagger_flag() && sp.T >= 16 * 1024) {
        const int nt = (sp.T + MMA_TILE - 1) / MMA_TILE;
        int n = std::max(2, (int)((3LL * nt * MMA_TILE) / (2LL * stagger_cap)));   // the longest chunk is about 1.5 means
        auto longest = [&](int nn) {
            int m = 0;
            for (int x = 0; x < nn; ++x) m = std::max(m, chunk_first_tile(x + 1, nn, nt) - chunk_first_tile(x, nn, nt));
            return m;
        };
        while (longest(n) * MMA_TILE > stagger_cap) ++n;
        if ((long long)rows * n <= cand_capacity_chunks(rows)) {
            stagger_tiles = nt;
            g1.x = (unsigned)n;
            tokens_per_cta = stagger_cap;
        }
    }
    ScoreParams sp2 = sp;
    AttendParams ap2 = ap;
    const int nchunks = (int)g1.x;
    const int kk = ap.top_k < sp.T ? ap.top_k : sp.T;
    size_t smem1 = 0;
    if (sp.T >= SKV_CAND_MIN_T && kk <= MAX_CAND_K && nchunks >= 2 && tokens_per_cta <= 8192 && (long long)nchunks * kk * 4 <= sp.T &&
        (long long)rows * nchunks <= cand_capacity_chunks(rows)) {
        sp2.cand_k = kk;
        sp2.cand_score = cand_base;
        sp2.cand_pos = reinterpret_cast<int*>(cand_base + cand_capacity_chunks(rows) * MAX_CAND_K);
        ap2.cand_score = sp2.cand_score;
        ap2.cand_pos = sp2.cand_pos;
        ap2.nc = nchunks * kk;
        smem1 = (size_t)tokens_per_cta * 4 + (size_t)TopkSmem<SCORE_THREADS>::WORDS * 4 + (size_t)MAX_CAND_K * 4;
        static bool configured1[64] = {false};
        if (device < 64 && !configured1[device]) {
            SKV_CUDA_TRY(cudaFuncSetAttribute(token_scores_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              8192 * 4 + (int)TopkSmem<SCORE_THREADS>::WORDS * 4 + MAX_CAND_K * 4));
            configured1[device] = true;
        }
    }
    bool scored = false;
    if constexpr (D == 64 || D == 128) {
        if (mma_path) {
            CUtensorMap tmK;
            KvMapPos pos;
            const int rc = make_kv_tmap(&tmK, &pos, sp.k, 2, 64, D / 64, B, sp.T, sp.H, sp.k_sb, sp.k_st, sp.k_sh, MMA_TILE);
            if (rc) return rc;
            // ring + the chunk's scores (candidate mode)
            const bool short_ring = tokens_per_cta <= 2048;
            const size_t ring_bytes = short_ring ? mma_ring_bytes<D, 2>() : mma_ring_bytes<D, 3>();
            const size_t smem_mma = 1024 + ring_bytes + (sp2.cand_k > 0 ? (size_t)tokens_per_cta * 4 : 0);
            static_assert((size_t)2 * mma_stage_bytes<D>() >= (size_t)TopkSmem<SCORE_THREADS>::WORDS * 4 + MAX_CAND_K * 4,
                          "the candidate select scratch lives in the drained ring");
            static int configured_mma[64][2] = {{0}};
            if (device < 64 && configured_mma[device][short_ring] < (int)smem_mma) {
                if (short_ring)
                    SKV_CUDA_TRY(cudaFuncSetAttribute(token_scores_mma_kernel<D, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_mma));
                else
                    SKV_CUDA_TRY(cudaFuncSetAttribute(token_scores_mma_kernel<D, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_mma));
                configured_mma[device][short_ring] = (int)smem_mma;
            }
            if (short_ring) token_scores_mma_kernel<D, 2><<<g1, SCORE_THREADS, smem_mma, st>>>(tmK, sp2, pos, tokens_per_cta, stagger_tiles, status);
            else token_scores_mma_kernel<D, 3><<<g1, SCORE_THREADS, smem_mma, st>>>(tmK, sp2, pos, tokens_per_cta, stagger_tiles, status);
            scored = true;
        }
    }
    if (!scored) token_scores_kernel<D><<<g1, SCORE_THREADS, smem1, st>>>(sp2, tokens_per_cta);
    SKV_CUDA_TRY(cudaGetLastError());
    SKV_CUDA_TRY(launch_pdl(token_select_attend_kernel<D>, dim3((unsigned)rows), dim3(ATT_THREADS), smem, st, ap2));
    SKV_CUDA_TRY(cudaGetLastError());
    return SKV_OK;
}

}  // namespace tsp
}  // namespace skv

using namespace skv;

extern "C" {

#ifdef SKV_PROFILE_PHASES
int skv_debug_phase_ts_token(unsigned long long* out) {
    return cudaMemcpyFromSymbol(out, skv_phase_ts, sizeof(unsigned long long) * 32) == cudaSuccess ? 0 : -4;
}
#endif

// 1 (default): decode-shaped calls (one query per head, D = 64 or 128) score the keys on the tensor cores; 0: always with
// the register-load kernel.  Process-wide.
int skv_token_sparse_set_mma_scores(int on) {
    tsp::mma_scores_flag() = on ? 1 : 0;
    return SKV_OK;
}

// 1 (default): the tensor-core scoring kernel's chunks have unequal lengths (1.5 to 0.5 times the mean along a row), so
// that the CTAs' candidate selections do not all fall into the same moments; 0: equal chunks.  Same results.  Process-wide.
int skv_token_sparse_set_stagger(int on) {
    tsp::stagger_flag() = on ? 1 : 0;
    return SKV_OK;
}

size_t skv_token_sparse_workspace_bytes(int B, int H, int S, int T) {
    if (B <= 0 || H <= 0 || S <= 0 || T <= 0) return 0;
    const size_t scores = (((size_t)B * H * S * T * sizeof(float)) + 255) & ~size_t(255);
    return 256 + scores + (size_t)tsp::cand_capacity_chunks((long long)B * H * S) * tsp::MAX_CAND_K * 8;
}

int skv_token_sparse_decode(const void* q, const void* k, const void* v, void* out, int* topk_idx_out,
                            void* workspace, size_t workspace_bytes, int B, int H, int S, int T, int D,
                            long long q_stride_b, long long q_stride_h, long long q_stride_s,
                            long long kv_stride_b, long long kv_stride_h, long long kv_stride_t,
                            int top_k, int sink_tokens, float scale, int device, void* stream) {
    if (!q || !k || !v || !out) return fail(SKV_ERR_BAD_ARG, "skv_token_sparse_decode: null tensor pointer");
    if (B <= 0 || H <= 0 || S <= 0 || T <= 0) return fail(SKV_ERR_BAD_ARG, "skv_token_sparse_decode: sizes must be positive");
    if (top_k <= 0) return fail(SKV_ERR_BAD_ARG, "top_k must be positive");
    if (sink_tokens < 0) return fail(SKV_ERR_BAD_ARG, "sink_tokens must not be negative");
    if (D != 16 && D != 32 && D != 64 && D != 128 && D != 256)
        return fail(SKV_ERR_UNSUPPORTED, "head dim %d not supported (16, 32, 64, 128 or 256)", D);
    const int kk = top_k < T ? top_k : T, sk = sink_tokens < T ? sink_tokens : T;
    if (kk + sk > tsp::MAX_KEEP)
        return fail(SKV_ERR_UNSUPPORTED, "top_k + sink_tokens = %d exceeds %d", kk + sk, tsp::MAX_KEEP);
    if (H > 65535 || (long long)B * S > 65535) return fail(SKV_ERR_UNSUPPORTED, "grid dimension too large");
    if ((kv_stride_t % 8) || (kv_stride_h % 8) || (kv_stride_b % 8) || (q_stride_b % 8) || (q_stride_h % 8) || (q_stride_s % 8))
        return fail(SKV_ERR_BAD_ARG, "strides must be multiples of 8 elements (16-byte rows)");
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15)
        return fail(SKV_ERR_BAD_ARG, "q/k/v must be 16-byte aligned");
    const size_t need = skv_token_sparse_workspace_bytes(B, H, S, T);
    if (!workspace || workspace_bytes < need)
        return fail(SKV_ERR_WORKSPACE, "workspace of %zu bytes is smaller than the %zu required", workspace_bytes, need);
    DeviceGuard guard(device);
    if (!guard.ok) return fail(SKV_ERR_CUDA, "cannot switch to device %d", device);

    tsp::ScoreParams sp;
    sp.q = static_cast<const __half*>(q);
    sp.k = static_cast<const __half*>(k);
    sp.scores = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + 256);
    sp.H = H; sp.S = S; sp.T = T;
    sp.q_sb = q_stride_b; sp.q_sh = q_stride_h; sp.q_ss = q_stride_s;
    sp.k_sb = kv_stride_b; sp.k_sh = kv_stride_h; sp.k_st = kv_stride_t;
    sp.scale = scale;
    sp.cand_score = nullptr; sp.cand_pos = nullptr; sp.cand_k = 0;
    tsp::AttendParams ap;
    ap.scores = sp.scores;
    ap.v = static_cast<const __half*>(v);
    ap.out = static_cast<__half*>(out);
    ap.topk_idx = topk_idx_out;
    ap.H = H; ap.S = S; ap.T = T; ap.top_k = top_k; ap.sink = sink_tokens;
    ap.v_sb = kv_stride_b; ap.v_sh = kv_stride_h; ap.v_st = kv_stride_t;
    ap.cand_score = nullptr; ap.cand_pos = nullptr; ap.nc = 0;
    const size_t scores_bytes = (((size_t)B * H * S * T * sizeof(float)) + 255) & ~size_t(255);
    float* cand_base = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + 256 + scores_bytes);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int* st_word = static_cast<int*>(workspace);   // the device status word sits at offset 0 of the workspace
    switch (D) {
        case 16: return tsp::launch<16>(sp, ap, B, device, st, cand_base, st_word);
        case 32: return tsp::launch<32>(sp, ap, B, device, st, cand_base, st_word);
        case 64: return tsp::launch<64>(sp, ap, B, device, st, cand_base, st_word);
        case 128: return tsp::launch<128>(sp, ap, B, device, st, cand_base, st_word);
        default: return tsp::launch<256>(sp, ap, B, device, st, cand_base, st_word);
    }
}

}  // extern "C"

SKV_BOUNDS_GETTER(skv_debug_bounds_token_sparse)
