// Block-sparse decode attention with the reference's block-mean rule.
//
// Replaces block_sparse_attn_kernel / sparse_attention_forward of the reference
// (csrc/kernels/sparse_attention.cu:26-175, :178-244; same arithmetic as
// jax_ref/sparse_attention_pallas.py:52-136):
//   s_j   = scale * mean_{t in block j} q . k_t        (ragged last block: its own count)
//   top-k blocks by s_j (equal scores: lower block first)
//   w     = softmax(s_top)
//   out   = sum_j w_j * mean_{t in block j} v_t
// The reference runs ONE WARP per (b, h) with a lane per block; here
//   1. block_mean_scores_kernel: a warp per block, D/8 lanes per key row, 16-byte
//      streaming loads over all of K (HBM-bound), per-lane partial sums reduced
//      once per block;
//   2. block_select_attend_kernel: a 1024-thread CTA per (b, h): exact top-k over
//      the block scores, softmax over k values, gather of k * block_size V rows.
#include "skv_common.cuh"
#include "skv_select.cuh"
#include "skv_tmap.cuh"

namespace skv {
namespace bsp {

constexpr int SCORE_THREADS = 256;
constexpr int ATT_THREADS = 1024;
constexpr int MAX_TOPK_BLOCKS = 4096;

struct ScoreParams {
    const __half* q;   // element (b,h,d) at b*q_sb + h*q_sh + d
    const __half* k;   // element (b,h,t,d) at b*k_sb + h*k_sh + t*k_st + d
    float* scores;     // [B, H, nb]
    int H, T, block_size, nb;
    long long q_sb, q_sh, k_sb, k_sh, k_st;
    float scale;
};

// grid (ceil(nb / blocks_per_cta), H, B)
template <int D>
__global__ void __launch_bounds__(SCORE_THREADS)
block_mean_scores_kernel(const ScoreParams p, int blocks_per_cta) {
    pdl_launch_dependents();  // the kernel that consumes these results may be scheduled now; it waits for this grid to finish
    constexpr int LPR = D / 8;
    constexpr int RPW = 32 / LPR;
    constexpr int U = 16;  // independent 16-byte loads in flight per lane
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane % LPR, rw = lane / LPR;
    const int h = blockIdx.y, b = blockIdx.z;
    float q[8];
    unpack8(*reinterpret_cast<const uint4*>(p.q + b * p.q_sb + h * p.q_sh + sub * 8), q);
    const __half* kbase = p.k + b * p.k_sb + h * p.k_sh + sub * 8;
    float* srow = p.scores + ((long long)b * p.H + h) * p.nb;
    const int j0 = blockIdx.x * blocks_per_cta, j1 = min(p.nb, j0 + blocks_per_cta);
    for (int j = j0 + warp; j < j1; j += SCORE_THREADS / 32) {
        const int t0 = j * p.block_size, t1 = min(p.T, t0 + p.block_size);
        float acc = 0.f, acc1 = 0.f;
        for (int base = t0; base < t1; base += U * RPW) {
            uint4 kv[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                // rows past the block's end are clamped to its last row and discarded below: unconditional loads
                // can all be issued before the first use
                const int t = min(base + u * RPW + rw, t1 - 1);
                kv[u] = ld_stream16(kbase + (long long)t * p.k_st);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) pin_loaded(kv[u]);
            float d[U];
#pragma unroll
            for (int u = 0; u < U; ++u) d[u] = base + u * RPW + rw < t1 ? dot8(kv[u], q) : 0.f;
#pragma unroll
            for (int w = U / 2; w > 0; w >>= 1)
#pragma unroll
                for (int u = 0; u < w; ++u) d[u] += d[u + w];
            acc += d[0];
        }
        acc = warp_sum(acc + acc1);
        if (lane == 0) srow[j] = acc * p.scale / (float)(t1 - t0);
    }
}

// Tensor-core variant of the scoring kernel (D = 64 or 128, block_size a multiple of 16).  The mean over a block of
// q . k_t is the sum of the tokens' scores divided by their count, so the keys stream exactly as in the token-sparse
// scoring kernel -- TMA boxes of 128 tokens x 64 channels into a 3-stage ring, one [128 tokens x D] . [D x 8] product per
// tile with the query in column 0 -- and each warp leaves the sum of its 16 tokens' scores in shared memory; when the
// CTA's chunk has streamed, every block adds its block_size / 16 partial sums in token order (the same order in every
// run).  Tokens past T read as zero.  Thread 0 refills a stage right after the block-wide barrier that ends its previous
// use; every wait is bounded, and one that runs out sets SKV_DEV_TIMEOUT and ends the CTA's loop.
// grid (ceil(nb / blocks_per_cta), H, B); blocks_per_cta * block_size is a multiple of 128
constexpr int MMA_TILE = 128;
constexpr int MMA_STAGES = 3;
template <int D>
__host__ __device__ constexpr int mma_stage_bytes() { return MMA_TILE * D * 2; }
template <int D>
__host__ __device__ constexpr size_t mma_ring_bytes() { return (size_t)MMA_STAGES * mma_stage_bytes<D>() + 64; }

template <int D>
__global__ void __launch_bounds__(SCORE_THREADS, 2)
block_mean_scores_mma_kernel(const __grid_constant__ CUtensorMap tmK, const ScoreParams p, const KvMapPos pos,
                             int blocks_per_cta, int* status) {
    pdl_launch_dependents();
    SKV_PHASE(0);
    constexpr int NH = D / 64, KSTEPS = D / 16, HALF_BYTES = MMA_TILE * 128, STAGE = mma_stage_bytes<D>();
    extern __shared__ uint8_t mma_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(mma_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t ring = smem_u32(smem);
    const uint32_t full_bar = ring + MMA_STAGES * STAGE;
    float* part16 = reinterpret_cast<float*>(smem + mma_ring_bytes<D>());   // sums of 16 tokens' scores, [chunk tokens / 16]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, tq = lane & 3, lj = lane >> 3, r8 = lane & 7;
    const int h = blockIdx.y, b = blockIdx.z;
    const int j0 = blockIdx.x * blocks_per_cta, j1 = min(p.nb, j0 + blocks_per_cta);
    const int t0 = j0 * p.block_size, t1 = min(p.T, j1 * p.block_size);
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
    uint32_t qb[KSTEPS][2];   // the query as the B operand: column 0 of the 8-wide N side, the other columns zero
    {
        const __half* qrow = p.q + b * p.q_sb + h * p.q_sh;
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {
            qb[kk][0] = g == 0 ? *reinterpret_cast<const uint32_t*>(qrow + kk * 16 + tq * 2) : 0u;
            qb[kk][1] = g == 0 ? *reinterpret_cast<const uint32_t*>(qrow + kk * 16 + 8 + tq * 2) : 0u;
        }
    }
    const uint32_t a_row_off = (uint32_t)((warp * 16 + (lj & 1) * 8 + r8) * 128);
    for (int i = 0; i < ntiles; ++i) {
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
            // column 0 (lanes tq == 0) holds the scores of tokens g and g + 8: sum the warp's 16 tokens over the 8 lanes g
            float v = tq == 0 ? (acc0[0] + acc1[0]) + (acc0[2] + acc1[2]) : 0.f;
            v += __shfl_xor_sync(0xffffffffu, v, 4);
            v += __shfl_xor_sync(0xffffffffu, v, 8);
            v += __shfl_xor_sync(0xffffffffu, v, 16);
            if (lane == 0) part16[i * (MMA_TILE / 16) + warp] = v;
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
            return;
        }
    }
    __syncthreads();
    SKV_PHASE(1);
    float* srow = p.scores + ((long long)b * p.H + h) * p.nb;
    const int per = p.block_size / 16;
    for (int j = j0 + tid; j < j1; j += SCORE_THREADS) {
        const int bt0 = j * p.block_size, bt1 = min(p.T, bt0 + p.block_size);
        float sum = 0.f;
        for (int u = 0; u < per; ++u) sum += part16[(j - j0) * per + u];   // (16-token groups past T hold zeros)
        srow[j] = sum * p.scale / (float)(bt1 - bt0);
    }
}

struct AttendParams {
    const float* scores;  // [rows, nb]
    const __half* v;
    __half* out;          // [rows, D]
    int* block_idx;       // optional [rows, top_k_blocks], ascending, -1 padded
    int H, T, block_size, nb, top_k;
    long long v_sb, v_sh, v_st;
};

// grid (B*H)
template <int D>
__global__ void __launch_bounds__(ATT_THREADS)
block_select_attend_kernel(const AttendParams p) {
    SKV_PHASE(3);
    pdl_wait_prior_grids();   // launched as a programmatic dependent of the scoring kernel: its results are complete from here on
    SKV_PHASE(4);
    constexpr int LPR = D / 8;
    constexpr int GROUPS = ATT_THREADS / LPR;
    extern __shared__ uint32_t dsm[];
    uint32_t* tk = dsm;
    int* sel = reinterpret_cast<int*>(tk + TopkSmem<ATT_THREADS>::WORDS);  // [MAX_TOPK_BLOCKS]
    float* w = reinterpret_cast<float*>(sel + MAX_TOPK_BLOCKS);            // [MAX_TOPK_BLOCKS]
    float* red = w + MAX_TOPK_BLOCKS;                                      // [GROUPS][D]
    __shared__ float bcast[2];

    const int row = blockIdx.x, h = row % p.H, b = row / p.H;
    const float* sc = p.scores + (long long)row * p.nb;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kk = min(p.top_k, p.nb);
    block_topk_fast<ATT_THREADS, 4>(sc, p.nb, kk, sel, tk);
    __syncthreads();
    SKV_PHASE(5);
    if (p.block_idx)
        for (int i = tid; i < p.top_k; i += ATT_THREADS) p.block_idx[(long long)row * p.top_k + i] = i < kk ? sel[i] : -1;

    // The value rows' addresses are known now, their weights only after the softmax: VU rows per thread are loaded
    // together (rows past the end are clamped to a real row and weighted zero, so no load waits on a condition), the
    // first batch before the softmax.
    constexpr int VU = 4;
    const int grp = tid / LPR, sub = tid % LPR;
    const __half* vbase = p.v + b * p.v_sb + h * p.v_sh + sub * 8;
    const int total = kk * p.block_size;   // gathered rows: at most T rounded up to a block, which the entry point keeps below 2^31
    auto row_token = [&](int r, int& i) {   // token of gathered row r (clamped), its block slot in i; < 0: past the end
        const int rc = r < total ? r : total - 1;
        i = rc / p.block_size;
        const int t = SKV_INDEX(sel[i], p.nb) * p.block_size + (rc - i * p.block_size);
        return (r < total && t < p.T) ? t : -1 - min(t, p.T - 1);
    };
    uint4 vraw[VU];
    int vslot[VU];
    auto load_batch = [&](int r0) {
#pragma unroll
        for (int u = 0; u < VU; ++u) {
            int i;
            const int t = row_token(r0 + u * GROUPS, i);
            vslot[u] = t >= 0 ? i : -1;
            vraw[u] = *reinterpret_cast<const uint4*>(vbase + (long long)(t >= 0 ? t : -1 - t) * p.v_st);
        }
    };
    if (total > 0) load_batch(grp);

    SKV_PHASE(6);
    // Up to 32 selected blocks (the usual case): every warp computes the k weights for itself, lane i holding block
    // i's, and hands them out by shuffle -- no shared memory and no block-wide barrier between selection and gather.
    const bool few = kk <= 32;
    float wlane = 0.f;
    if (few) {
        const float x = lane < kk ? sc[SKV_INDEX(sel[lane], p.nb)] : -INFINITY;
        const float mxw = warp_max(x);
        const float e = lane < kk ? __expf(x - mxw) : 0.f;
        const float inv = 1.f / fmaxf(warp_sum(e), 1e-9f);
        if (lane < kk) {
            const int t0 = SKV_INDEX(sel[lane], p.nb) * p.block_size;
            wlane = e * inv / (float)(min(p.T, t0 + p.block_size) - t0);
        }
    }
    // softmax over the kk selected block scores, folded with 1 / count of each block
    float mx = -INFINITY;
    if (!few) {
    for (int i = tid; i < kk; i += ATT_THREADS) {
        const float x = sc[SKV_INDEX(sel[i], p.nb)];
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
    for (int i = tid; i < kk; i += ATT_THREADS) {
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
    const float inv = 1.f / fmaxf(bcast[1], 1e-9f);
    for (int i = tid; i < kk; i += ATT_THREADS) {
        const int t0 = SKV_INDEX(sel[i], p.nb) * p.block_size;
        const int cnt = min(p.T, t0 + p.block_size) - t0;
        w[i] = w[i] * inv / (float)cnt;  // per-token weight of block i
    }
    __syncthreads();
    }

    SKV_PHASE(7);
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int base = 0; base < total; base += VU * GROUPS) {   // (the same trip count in every thread: the shuffles below need whole warps; rows past the end weigh zero)
        if (base) load_batch(base + grp);
#pragma unroll
        for (int u = 0; u < VU; ++u) {
            float x[8];
            unpack8(vraw[u], x);
            float wi;
            if (few) {
                const float ws = __shfl_sync(0xffffffffu, wlane, max(vslot[u], 0));
                wi = vslot[u] >= 0 ? ws : 0.f;
            } else {
                wi = vslot[u] >= 0 ? w[vslot[u]] : 0.f;
            }
#pragma unroll
            for (int c = 0; c < 8; ++c) acc[c] = fmaf(wi, x[c], acc[c]);
        }
    }
    SKV_PHASE(8);
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 8; ++i) red[grp * D + sub * 8 + i] = acc[i];
    __syncthreads();
    for (int d = tid; d < D; d += ATT_THREADS) {
        float o = 0.f;
#pragma unroll 8
        for (int g2 = 0; g2 < GROUPS; ++g2) o += red[g2 * D + d];
        p.out[(long long)row * D + d] = __float2half_rn(o);
    }
    SKV_PHASE(9);
}

// 1 (default): D = 64 or 128 with block sizes that are multiples of 16 are scored by the tensor-core kernel; 0: always
// the register-load kernel.
inline int& mma_scores_flag() { static int on = 1; return on; }

template <int D>
static int launch(const ScoreParams& sp, const AttendParams& ap, int B, int device, cudaStream_t st, int* status) {
    static bool configured[64] = {false};
    const size_t smem = (size_t)TopkSmem<ATT_THREADS>::WORDS * 4 + (size_t)MAX_TOPK_BLOCKS * 8 +
                        (size_t)(ATT_THREADS / (D / 8)) * D * 4;
    if (device < 64 && !configured[device]) {
        SKV_CUDA_TRY(cudaFuncSetAttribute(block_select_attend_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured[device] = true;
    }
    const long long rows = (long long)B * sp.H;
    long long want = ((long long)sm_count(device) * 8 + rows - 1) / rows;  // CTAs per (b, h)
    int blocks_per_cta = (int)((sp.nb + want - 1) / want);
    const int warps = SCORE_THREADS / 32;
    blocks_per_cta = ((blocks_per_cta + warps - 1) / warps) * warps;
    dim3 g1((sp.nb + blocks_per_cta - 1) / blocks_per_cta, sp.H, B);
    bool scored = false;
    if constexpr (D == 64 || D == 128) {
        if (mma_scores_flag() && sp.block_size % 16 == 0 && sp.block_size <= 1024) {
            // chunks of whole 128-token tiles (so that a 16-token group never belongs to two CTAs), at most 16 K tokens
            // blocks per chunk: a multiple of the fewest whole blocks that make whole 128-token tiles
            int gcd = MMA_TILE, r = sp.block_size % MMA_TILE;
            while (r) { const int t = gcd % r; gcd = r; r = t; }
            const int unit = MMA_TILE / gcd;
            int bpc = ((blocks_per_cta + unit - 1) / unit) * unit;
            const int max_bpc = (16384 / sp.block_size) / unit * unit;
            if (bpc > max_bpc) bpc = max_bpc;
            if (bpc >= unit && (long long)bpc * sp.block_size % MMA_TILE == 0) {
                CUtensorMap tmK;
                KvMapPos pos;
                const int rc = make_kv_tmap(&tmK, &pos, sp.k, 2, 64, D / 64, B, sp.T, sp.H, sp.k_sb, sp.k_st, sp.k_sh, MMA_TILE);
                if (rc) return rc;
                const size_t smem_mma = 1024 + mma_ring_bytes<D>() + (size_t)bpc * sp.block_size / 16 * 4;
                static int configured_mma[64] = {0};
                if (device < 64 && configured_mma[device] < (int)smem_mma) {
                    SKV_CUDA_TRY(cudaFuncSetAttribute(block_mean_scores_mma_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_mma));
                    configured_mma[device] = (int)smem_mma;
                }
                dim3 g2((sp.nb + bpc - 1) / bpc, sp.H, B);
                block_mean_scores_mma_kernel<D><<<g2, SCORE_THREADS, smem_mma, st>>>(tmK, sp, pos, bpc, status);
                scored = true;
            }
        }
    }
    if (!scored) block_mean_scores_kernel<D><<<g1, SCORE_THREADS, 0, st>>>(sp, blocks_per_cta);
    SKV_CUDA_TRY(cudaGetLastError());
    SKV_CUDA_TRY(launch_pdl(block_select_attend_kernel<D>, dim3((unsigned)rows), dim3(ATT_THREADS), smem, st, ap));
    SKV_CUDA_TRY(cudaGetLastError());
    return SKV_OK;
}

}  // namespace bsp
}  // namespace skv

using namespace skv;

extern "C" {

#ifdef SKV_PROFILE_PHASES
int skv_debug_phase_ts_block(unsigned long long* out) {
    return cudaMemcpyFromSymbol(out, skv_phase_ts, sizeof(unsigned long long) * 32) == cudaSuccess ? 0 : -4;
}
#endif

// 1 (default): D = 64 or 128 with a block size that is a multiple of 16 scores the blocks on the tensor cores; 0: always
// with the register-load kernel.  Process-wide.
int skv_block_sparse_set_mma_scores(int on) {
    bsp::mma_scores_flag() = on ? 1 : 0;
    return SKV_OK;
}

size_t skv_block_sparse_workspace_bytes(int B, int H, int T, int block_size) {
    if (B <= 0 || H <= 0 || T <= 0 || block_size <= 0) return 0;
    const size_t nb = ((size_t)T + block_size - 1) / block_size;
    return 256 + (((size_t)B * H * nb * sizeof(float) + 255) & ~size_t(255));
}

int skv_block_sparse_decode(const void* q, const void* k, const void* v, void* out, int* block_idx_out,
                            void* workspace, size_t workspace_bytes, int B, int H, int T, int D,
                            long long q_stride_b, long long q_stride_h,
                            long long kv_stride_b, long long kv_stride_h, long long kv_stride_t,
                            int block_size, int top_k_blocks, float scale, int device, void* stream) {
    if (!q || !k || !v || !out) return fail(SKV_ERR_BAD_ARG, "skv_block_sparse_decode: null tensor pointer");
    if (B <= 0 || H <= 0 || T <= 0) return fail(SKV_ERR_BAD_ARG, "skv_block_sparse_decode: sizes must be positive");
    if (top_k_blocks <= 0) return fail(SKV_ERR_BAD_ARG, "top_k_blocks must be positive");
    if (block_size <= 0) return fail(SKV_ERR_BAD_ARG, "block_size must be positive");
    if (D != 16 && D != 32 && D != 64 && D != 128 && D != 256)
        return fail(SKV_ERR_UNSUPPORTED, "head dim %d not supported (16, 32, 64, 128 or 256)", D);
    const int nb = (T + block_size - 1) / block_size;
    if ((long long)nb * block_size > 2147483647LL)
        return fail(SKV_ERR_UNSUPPORTED, "skv_block_sparse_decode: T rounded up to a block must stay below 2^31");
    if ((top_k_blocks < nb ? top_k_blocks : nb) > bsp::MAX_TOPK_BLOCKS)
        return fail(SKV_ERR_UNSUPPORTED, "top_k_blocks=%d exceeds %d", top_k_blocks, bsp::MAX_TOPK_BLOCKS);
    if (H > 65535 || B > 65535) return fail(SKV_ERR_UNSUPPORTED, "grid dimension too large");
    if ((kv_stride_t % 8) || (kv_stride_h % 8) || (kv_stride_b % 8) || (q_stride_b % 8) || (q_stride_h % 8))
        return fail(SKV_ERR_BAD_ARG, "strides must be multiples of 8 elements (16-byte rows)");
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15)
        return fail(SKV_ERR_BAD_ARG, "q/k/v must be 16-byte aligned");
    const size_t need = skv_block_sparse_workspace_bytes(B, H, T, block_size);
    if (!workspace || workspace_bytes < need)
        return fail(SKV_ERR_WORKSPACE, "workspace of %zu bytes is smaller than the %zu required", workspace_bytes, need);
    DeviceGuard guard(device);
    if (!guard.ok) return fail(SKV_ERR_CUDA, "cannot switch to device %d", device);

    bsp::ScoreParams sp;
    sp.q = static_cast<const __half*>(q);
    sp.k = static_cast<const __half*>(k);
    sp.scores = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + 256);
    sp.H = H; sp.T = T; sp.block_size = block_size; sp.nb = nb;
    sp.q_sb = q_stride_b; sp.q_sh = q_stride_h;
    sp.k_sb = kv_stride_b; sp.k_sh = kv_stride_h; sp.k_st = kv_stride_t;
    sp.scale = scale;
    bsp::AttendParams ap;
    ap.scores = sp.scores;
    ap.v = static_cast<const __half*>(v);
    ap.out = static_cast<__half*>(out);
    ap.block_idx = block_idx_out;
    ap.H = H; ap.T = T; ap.block_size = block_size; ap.nb = nb; ap.top_k = top_k_blocks;
    ap.v_sb = kv_stride_b; ap.v_sh = kv_stride_h; ap.v_st = kv_stride_t;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int* st_word = static_cast<int*>(workspace);   // the device status word sits at offset 0 of the workspace
    switch (D) {
        case 16: return bsp::launch<16>(sp, ap, B, device, st, st_word);
        case 32: return bsp::launch<32>(sp, ap, B, device, st, st_word);
        case 64: return bsp::launch<64>(sp, ap, B, device, st, st_word);
        case 128: return bsp::launch<128>(sp, ap, B, device, st, st_word);
        default: return bsp::launch<256>(sp, ap, B, device, st, st_word);
    }
}

}  // extern "C"

SKV_BOUNDS_GETTER(skv_debug_bounds_block_sparse)
