// Quest-style block-sparse decode over a paged 8-bit KV cache.
//
// No reference counterpart: the reference's block-sparse kernel scores blocks by
// the mean of q.k over all keys of an unpaged fp16 cache
// (csrc/kernels/sparse_attention.cu:51-78).  Here, per block of `block_size`
// tokens and kv-head, the channel-wise min and max of the dequantised keys are
// kept as metadata; a block's score for a query head is the upper bound
//     scale * sum_d max(q_d * min_d, q_d * max_d)
// of scale * q.k over the block; the top_k_blocks best blocks are chosen per
// QUERY head (ties: lower block) and exact softmax attention runs over the tokens
// of the chosen blocks only, gathered page by page.
//
// Kernels:
//   block_meta_build_kernel  -- cache maintenance: one warp per (b, kv-head,
//       block) reads the block's codes and scales once and writes min|max fp16.
//   quest_scores_kernel      -- streams the metadata (HBM-bound), D/8 lanes per
//       block, all G query heads of the group scored from one read.
//   quest_select_attend_kernel -- one CTA per (b, query head): exact top-k over
//       the block scores, then scores / softmax / weighted value sum over the
//       <= k * block_size gathered tokens, all fp32; the V rows travel to shared
//       memory as asynchronous copies while the K rows are scored.
#include <cstring>

#include <cuda_fp8.h>

#include "skv_common.cuh"
#include "skv_select.cuh"
#include "skv_tmap.cuh"

namespace skv {
namespace quest {

constexpr int D = 128;
constexpr int META_THREADS = 256;
constexpr int SCORE_THREADS = 256;
constexpr int ATT_THREADS = 512;
constexpr int MAX_SEL_TOKENS = 2048;  // top_k_blocks * block_size upper bound
constexpr int MAX_TOPK = 256;
constexpr int PAST_END = 1 << 30;  // flag in the slot word of a gathered token that lies past the sequence end

template <int KVT>
__device__ __forceinline__ float code_to_float(uint32_t byte) {
    if (KVT == SKV_KV_E4M3) {
        const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)byte, __NV_E4M3);
        return __half2float(*reinterpret_cast<const __half*>(&h));
    }
    return (float)(int)(int8_t)byte;
}

// Four codes of one 32-bit word as floats.
template <int KVT>
__device__ __forceinline__ void word_to_floats(uint32_t w, float (&f)[4]) {
    if (KVT == SKV_KV_E4M3) {
        uint32_t h0, h1;
        asm("{\n\t.reg .b16 a, b;\n\tmov.b32 {a, b}, %2;\n\t"
            "cvt.rn.f16x2.e4m3x2 %0, a;\n\tcvt.rn.f16x2.e4m3x2 %1, b;\n\t}"
            : "=r"(h0), "=r"(h1)
            : "r"(w));
        const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&h0));
        const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&h1));
        f[0] = f0.x; f[1] = f0.y; f[2] = f1.x; f[3] = f1.y;
    } else {
        // int8 b -> float: the bits 0x4B000000 | (b ^ 0x80) are 2^23 + b + 128 exactly
        const uint32_t x = w ^ 0x80808080u;
#pragma unroll
        for (int i = 0; i < 4; ++i) f[i] = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7540u + i)) - 8388736.f;
    }
}

// Sixteen codes of one 16-byte load as floats.  FP8 goes through the paired conversion (one instruction per two
// codes): converting byte by byte made the gather kernel wait on the conversion pipe rather than on memory.
template <int KVT>
__device__ __forceinline__ void unpack16(const uint4& raw, float (&x)[16]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float f[4];
        word_to_floats<KVT>(w[i], f);
#pragma unroll
        for (int j = 0; j < 4; ++j) x[4 * i + j] = f[j];
    }
}

// Sixteen 4-bit value codes (eight bytes: channel 2j in the low, 2j+1 in the high nibble of byte j; nibble = code + 8)
__device__ __forceinline__ void unpack16_v4(const uint2& raw, float (&x)[16]) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t w = j < 4 ? raw.x : raw.y;
        const uint32_t byte = (w >> (8 * (j & 3))) & 0xFFu;
        x[2 * j] = (float)(int)(byte & 15u) - 8.f;
        x[2 * j + 1] = (float)(int)(byte >> 4) - 8.f;
    }
}

struct Pool {
    const uint8_t* codes;   // element (page,h,slot,d) at page*sp + h*sh + slot*ss + d
    const float* scales;    // element (page,h,slot) at page*csp + h*csh + slot
    long long sp, sh, ss, csp, csh;
};

struct MetaParams {
    Pool k;
    const int* page_table;  // [B, max_pages] or null
    const int* seq_lens;    // [B] or null
    __half* meta;           // [B, Hkv, nb, 2, D]
    int* status;            // optional device status word (SKV_DEV_BAD_PAGE)
    int B, Hkv, N, nb, block_size, page_size, max_pages, num_pages;
};

__device__ __forceinline__ int phys_page(const int* page_table, int b, int max_pages, int lp) {
    return page_table ? __ldg(page_table + (long long)b * max_pages + lp) : b * max_pages + lp;
}

// one warp per (b, h, block); lanes: 8 per token row (16 codes each), 4 rows per step.  The dequantised value
// code * scale is formed in fp32 and rounded to fp16 BEFORE the comparisons (rounding is monotone, so the minimum
// of the rounded values is the rounded minimum): minima and maxima then run two channels per instruction.
template <int KVT>
__global__ void __launch_bounds__(META_THREADS, 4)   // 64 registers: four CTAs per SM keep enough rows in flight
block_meta_build_kernel(const MetaParams p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane & 7, rw = lane >> 3;
    const long long total = (long long)p.B * p.Hkv * p.nb;
    bool bad_page = false;
    for (long long item = (long long)blockIdx.x * (META_THREADS / 32) + warp; item < total;
         item += (long long)gridDim.x * (META_THREADS / 32)) {
        const int blk = (int)(item % p.nb);
        const int h = (int)((item / p.nb) % p.Hkv);
        const int b = (int)(item / ((long long)p.nb * p.Hkv));
        const int len = p.seq_lens ? min(max(p.seq_lens[b], 0), p.N) : p.N;
        const int t0 = blk * p.block_size, t1 = min(len, t0 + p.block_size);
        __half2 lo[8], hi[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            lo[i] = __float2half2_rn(INFINITY);
            hi[i] = __float2half2_rn(-INFINITY);
        }
        constexpr int RU = 4;  // rows per lane group and step: page ids, then codes and scales, all issued together
        for (int tb = t0 + rw; tb < t1; tb += 4 * RU) {
            // Rows past the block's end are clamped to its last row: a repeated row changes no minimum or maximum,
            // and loads without a condition are all issued before the first use.
            int page[RU], slot[RU];
#pragma unroll
            for (int u = 0; u < RU; ++u) {
                const int t = min(tb + 4 * u, t1 - 1);
                const int lp = t / p.page_size;
                slot[u] = t - lp * p.page_size;
                page[u] = checked_page(phys_page(p.page_table, b, p.max_pages, lp), p.num_pages, bad_page);
            }
            uint4 raw[RU];
            float sc[RU];
#pragma unroll
            for (int u = 0; u < RU; ++u) {
                raw[u] = ld_stream16(p.k.codes + page[u] * p.k.sp + h * p.k.sh + slot[u] * p.k.ss + sub * 16);
                sc[u] = __ldg(p.k.scales + page[u] * p.k.csp + h * p.k.csh + slot[u]);
            }
#pragma unroll
            for (int u = 0; u < RU; ++u) {
                const uint32_t w[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float f[4];
                    word_to_floats<KVT>(w[j], f);
                    const __half2 v0 = __floats2half2_rn(f[0] * sc[u], f[1] * sc[u]);
                    const __half2 v1 = __floats2half2_rn(f[2] * sc[u], f[3] * sc[u]);
                    lo[2 * j] = __hmin2(lo[2 * j], v0);
                    hi[2 * j] = __hmax2(hi[2 * j], v0);
                    lo[2 * j + 1] = __hmin2(lo[2 * j + 1], v1);
                    hi[2 * j + 1] = __hmax2(hi[2 * j + 1], v1);
                }
            }
        }
        uint32_t wlo[8], whi[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
#pragma unroll
            for (int o = 8; o <= 16; o <<= 1) {
                const uint32_t a = __shfl_xor_sync(0xffffffffu, *reinterpret_cast<uint32_t*>(&lo[i]), o);
                const uint32_t c = __shfl_xor_sync(0xffffffffu, *reinterpret_cast<uint32_t*>(&hi[i]), o);
                lo[i] = __hmin2(lo[i], *reinterpret_cast<const __half2*>(&a));
                hi[i] = __hmax2(hi[i], *reinterpret_cast<const __half2*>(&c));
            }
            wlo[i] = *reinterpret_cast<uint32_t*>(&lo[i]);
            whi[i] = *reinterpret_cast<uint32_t*>(&hi[i]);
        }
        if (rw < 2) {  // row-group 0 writes the mins, row-group 1 the maxes
            __half* dst = p.meta + (item * 2 + rw) * D + sub * 16;
            const uint32_t* w = rw == 0 ? wlo : whi;
            *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
            *reinterpret_cast<uint4*>(dst + 8) = make_uint4(w[4], w[5], w[6], w[7]);
        }
    }
    report_bad_page(bad_page, p.status);
}

struct ScoreParams {
    const __half* q;      // [B, Hq, D]
    const __half* meta;   // [B, Hkv, nb, 2, D]
    float* scores;        // [B, Hq, nb]
    int Hq, Hkv, G, nb;
    float scale;
};

// 16 lanes per block (8 channels each), 2 blocks per warp-wide load, U loads of each half in flight per lane.
// With lo <= hi, max(q*lo, q*hi) = q*(hi+lo)/2 + |q|*(hi-lo)/2; hi+lo and hi-lo are exact in fp32 (fp16 inputs), the
// halving is folded into q, and |q| is an operand modifier of the FMA, so a channel costs two FMAs per head and the
// query needs one register per channel and head.  That leaves room for up to 8 blocks (sixteen 16-byte loads) in
// flight per lane at 128 registers: two CTAs per SM then keep 128 KB of metadata in flight per SM.
//
// Schedule: the (b, kv-head, block) space is flattened and cut into one contiguous range per WARP of a grid of exactly
// two CTAs per SM (blocks_per_warp, a multiple of 2U, chosen on the host so that the ranges cover the space with the
// least idle tail -- the kernel is a single wave and its duration is that of its slowest SM).  A range may cross
// into the next (b, kv-head): the query registers are reloaded there.
template <int MAXG, int U>
__global__ void __launch_bounds__(SCORE_THREADS, 2)
quest_scores_kernel(const ScoreParams p, long long total_blocks, int blocks_per_warp) {
    pdl_launch_dependents();  // the kernel that consumes these results may be scheduled now; it waits for this grid to finish
    static_assert(MAXG == 4 || MAXG == 8, "the packed reduction below is written for 4 or 8 heads");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane & 15, rw = lane >> 4;
    const long long gw = (long long)blockIdx.x * (SCORE_THREADS / 32) + warp;
    long long g0 = gw * blocks_per_warp;
    const long long g1 = min(total_blocks, g0 + blocks_per_warp);
    while (g0 < g1) {
        const long long row = g0 / p.nb;            // (b, kv-head)
        const int j0 = (int)(g0 - row * p.nb);
        const int j1 = (int)min((long long)p.nb, j0 + (g1 - g0));
        const int b = (int)(row / p.Hkv), h = (int)(row - (long long)b * p.Hkv);
        float qh[MAXG][8];   // half the query
#pragma unroll
        for (int g = 0; g < MAXG; ++g) {
            float q[8];
            if (g < p.G) unpack8(*reinterpret_cast<const uint4*>(p.q + ((long long)b * p.Hq + h * p.G + g) * D + sub * 8), q);
            else
#pragma unroll
                for (int i = 0; i < 8; ++i) q[i] = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) qh[g][i] = 0.5f * q[i];
        }
        const __half* mbase = p.meta + row * p.nb * 2 * D + sub * 8;
        for (int base = j0; base < j1; base += 2 * U) {
            uint4 lo4[U], hi4[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int j = min(base + u * 2 + rw, j1 - 1);  // clamped; the store below is guarded
                lo4[u] = ld_stream16(mbase + (long long)j * 2 * D);
                hi4[u] = ld_stream16(mbase + (long long)j * 2 * D + D);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int j = base + u * 2 + rw;
                float lo[8], hi[8], acc[MAXG];
                unpack8(lo4[u], lo);
                unpack8(hi4[u], hi);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float s = hi[i] + lo[i], d = hi[i] - lo[i];
                    lo[i] = s;   // hi + lo
                    hi[i] = d;   // hi - lo >= 0
                }
#pragma unroll
                for (int g = 0; g < MAXG; ++g) {
                    acc[g] = 0.f;
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[g] = fmaf(qh[g][i], lo[i], fmaf(fabsf(qh[g][i]), hi[i], acc[g]));
                }
                // Sum over the 16 lanes of the half-warp, several heads at once: at each of the first steps a lane
                // keeps half of its values and hands the other half to its partner, so MAXG values cost
                // MAXG/2 + MAXG/4 + ... + 1 shuffles plus the remaining plain steps instead of 4 * MAXG.
                int head = 0;  // which head this lane ends up holding
                float v4[4];
                if (MAXG == 8) {
                    const bool up = sub & 8;
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const float keep = up ? acc[g + 4] : acc[g], send = up ? acc[g] : acc[g + 4];
                        v4[g] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
                    }
                    head = up ? 4 : 0;
                } else {
#pragma unroll
                    for (int g = 0; g < 4; ++g) v4[g] = acc[g] + __shfl_xor_sync(0xffffffffu, acc[g], 8);
                }
                float v2[2];
                {
                    const bool up = sub & 4;
#pragma unroll
                    for (int g = 0; g < 2; ++g) {
                        const float keep = up ? v4[g + 2] : v4[g], send = up ? v4[g] : v4[g + 2];
                        v2[g] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
                    }
                    head += up ? 2 : 0;
                }
                float v1;
                {
                    const bool up = sub & 2;
                    const float keep = up ? v2[1] : v2[0], send = up ? v2[0] : v2[1];
                    v1 = keep + __shfl_xor_sync(0xffffffffu, send, 2);
                    head += up ? 1 : 0;
                }
                v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
                if (j < j1 && (sub & 1) == 0 && head < p.G)
                    p.scores[((long long)b * p.Hq + h * p.G + head) * p.nb + j] = v1 * p.scale;
            }
        }
        g0 += j1 - j0;
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Tensor-core variant of the scoring kernel (see skv_quest_set_ring_scores).  With lo <= hi,
//     sum_c max(q_c lo_c, q_c hi_c) = sum_c min(q_c, 0) lo_c + sum_c max(q_c, 0) hi_c,
// i.e. the score of a block is one dot product of its 256 stored numbers (128 minima, then 128 maxima) with the
// 256-vector (min(q, 0) | max(q, 0)): scoring is a [blocks x 256] . [256 x heads] product, and the register-load
// kernel's ~120 instructions per block and lane become 16 MMAs per 16 blocks.  The metadata then streams like K in
// the dense decode kernel: one persistent CTA per SM takes a contiguous range of (row, 64-block tile) items, a
// producer lane issues four TMA boxes per tile ([64 blocks][64 numbers], 128-byte swizzle, evict-first) into a
// 5-stage ring, four consumer warps take 16 blocks each (ldmatrix + mma.sync.m16n8k16, blocks on the M side, up to 8
// query heads on the N side).  A tile never spans two (b, kv-head) rows; what a box reads past the end of its row is
// computed and not stored.  Every wait is bounded; one that runs out sets SKV_DEV_TIMEOUT and the CTA stops.
// ---------------------------------------------------------------------------------------------------------------
constexpr int MS_TILE = 64;                               // blocks per stage
constexpr int MS_BOX_BYTES = MS_TILE * 128;               // one [64][64 halves] box
constexpr int MS_STAGE_BYTES = 4 * MS_BOX_BYTES;          // 32 KB
constexpr int MS_STAGES = 5;
constexpr int MS_CONSUMER_WARPS = 4;
constexpr int MS_THREADS = (MS_CONSUMER_WARPS + 1) * 32;
constexpr size_t MS_SMEM = (size_t)MS_STAGES * MS_STAGE_BYTES + 2 * MS_STAGES * 8 + 1024;

__global__ void __launch_bounds__(MS_THREADS, 1)
quest_scores_mma_kernel(const __grid_constant__ CUtensorMap tmM, const ScoreParams p, int tiles_per_row,
                        long long total_items, long long items_per_cta, int* status) {
    pdl_launch_dependents();  // the kernel that consumes these results may be scheduled now; it waits for this grid to finish
    extern __shared__ uint8_t ms_raw[];
    uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(ms_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t ring_u32 = smem_u32(ring);
    const uint32_t full_bar = ring_u32 + MS_STAGES * MS_STAGE_BYTES, empty_bar = full_bar + MS_STAGES * 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long i0 = min(total_items, (long long)blockIdx.x * items_per_cta);
    const long long i1 = min(total_items, i0 + items_per_cta);
    if (threadIdx.x == 0) {
        for (int s = 0; s < MS_STAGES; ++s) {
            mbar_init(full_bar + s * 8, 1);
            mbar_init(empty_bar + s * 8, MS_CONSUMER_WARPS);
        }
        fence_barrier_init();
    }
    __syncthreads();
    int row = (int)(i0 / tiles_per_row), tile = (int)(i0 - (long long)row * tiles_per_row);

    if (warp == MS_CONSUMER_WARPS) {   // producer: one lane, four boxes per tile
        if (lane == 0) {
            tma_prefetch_desc(&tmM);
            const uint64_t policy = l2_policy_evict_first();
            int s = 0;
            uint32_t ph = 0;
            long long n = 0;
            for (long long it = i0; it < i1; ++it, ++n) {
                if (n >= MS_STAGES && !mbar_wait(empty_bar + s * 8, ph ^ 1u)) {
                    atomicOr(status, SKV_DEV_TIMEOUT);
                    break;
                }
                const uint32_t dst = ring_u32 + s * MS_STAGE_BYTES, bar = full_bar + s * 8;
                mbar_expect_tx(bar, MS_STAGE_BYTES);
                const int first = row * p.nb + tile * MS_TILE;      // first block (a row of the [blocks][256] matrix)
#pragma unroll
                for (int hf = 0; hf < 4; ++hf) tma_load_2d(dst + hf * MS_BOX_BYTES, &tmM, bar, hf * 64, first, policy);
                if (++s == MS_STAGES) { s = 0; ph ^= 1u; }
                if (++tile == tiles_per_row) { tile = 0; ++row; }
            }
        }
        return;
    }

    // consumers: warp w scores blocks 16w .. 16w+15 of every tile; lane (g, tq) ends up with blocks g and g+8 for heads
    // 2tq and 2tq+1
    const int g = lane >> 2, tq = lane & 3;
    const int lj = lane >> 3, r8 = lane & 7;
    const uint32_t a_row_off = (uint32_t)((warp * 16 + (lj & 1) * 8 + r8) * 128);   // this lane's ldmatrix row (row & 7 == r8)
    uint32_t qb[16][2];    // B operand: k-steps 0..7 hold min(q, 0) (against the minima), 8..15 max(q, 0)
    int cur_row = -1;
    int s = 0;
    uint32_t ph = 0;
    for (long long it = i0; it < i1; ++it) {
        if (row != cur_row) {
            cur_row = row;
            const __half* qrow = p.q + ((long long)row * p.G + g) * D;
            const __half2 zero = __float2half2_rn(0.f);
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                __half2 u = zero, v = zero;
                if (g < p.G) {
                    u = *reinterpret_cast<const __half2*>(qrow + kk * 16 + tq * 2);
                    v = *reinterpret_cast<const __half2*>(qrow + kk * 16 + 8 + tq * 2);
                }
                const __half2 un = __hmin2(u, zero), vn = __hmin2(v, zero), up = __hmax2(u, zero), vp = __hmax2(v, zero);
                qb[kk][0] = *reinterpret_cast<const uint32_t*>(&un);
                qb[kk][1] = *reinterpret_cast<const uint32_t*>(&vn);
                qb[kk + 8][0] = *reinterpret_cast<const uint32_t*>(&up);
                qb[kk + 8][1] = *reinterpret_cast<const uint32_t*>(&vp);
            }
        }
        int ok = 1;
        if (lane == 0) ok = mbar_wait(full_bar + s * 8, ph) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) {
            if (lane == 0) atomicOr(status, SKV_DEV_TIMEOUT);
            return;
        }
        const uint32_t base = ring_u32 + s * MS_STAGE_BYTES + a_row_off;
        float acc0[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};   // even / odd k-steps: half the dependent chain
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
            const int c = 2 * kk + (lj >> 1);        // 16-byte chunk of the block's 512 bytes
            uint32_t a[4];
            ldsm_x4(base + (uint32_t)(c >> 3) * MS_BOX_BYTES + (uint32_t)(((c & 7) ^ r8) << 4), a[0], a[1], a[2], a[3]);
            if (kk & 1) mma_f16(acc1, a, qb[kk][0], qb[kk][1]);
            else mma_f16(acc0, a, qb[kk][0], qb[kk][1]);
        }
        const int j = tile * MS_TILE + warp * 16 + g;
        float* dst = p.scores + ((long long)row * p.G + tq * 2) * p.nb + j;
        if (tq * 2 < p.G) {
            if (j < p.nb) dst[0] = (acc0[0] + acc1[0]) * p.scale;
            if (j + 8 < p.nb) dst[8] = (acc0[2] + acc1[2]) * p.scale;
        }
        if (tq * 2 + 1 < p.G) {
            if (j < p.nb) dst[p.nb] = (acc0[1] + acc1[1]) * p.scale;
            if (j + 8 < p.nb) dst[p.nb + 8] = (acc0[3] + acc1[3]) * p.scale;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar + s * 8);
        if (++s == MS_STAGES) { s = 0; ph ^= 1u; }
        if (++tile == tiles_per_row) { tile = 0; ++row; }
    }
}

inline int& fused_flag() { static int on = 0; return on; }   // 1: score inside the attend kernel (clusters of G CTAs); measures the same (config 4: 38.9 against 38.0 us)
inline int& ring_scores_flag() { static int on = 1; return on; }   // tensor-core scoring: config 4 end to end 46 -> 40 us
inline bool use_ring_scores() { return ring_scores_flag() != 0; }

template <int MAXG, int U>
static cudaError_t launch_scores(const ScoreParams& sp, long long total_blocks, int blocks_per_warp, int ctas, cudaStream_t st) {
    quest_scores_kernel<MAXG, U><<<(unsigned)ctas, SCORE_THREADS, 0, st>>>(sp, total_blocks, blocks_per_warp);
    return cudaGetLastError();
}

struct AttendParams {
    const __half* q;       // [B, Hq, D]
    const float* scores;   // [B, Hq, nb]
    Pool k, v;
    const int* page_table;
    const int* seq_lens;
    __half* out;           // [B, Hq, D]
    int* block_idx;        // optional [B, Hq, top_k]
    int* status;           // device status word (SKV_DEV_BAD_PAGE)
    int Hq, G, N, nb, block_size, page_size, max_pages, num_pages, top_k;
    int v4;                // V rows hold 4-bit codes, 64 bytes per token (mixed-precision page records; v.ss = 64)
    float scale;
};

constexpr int VSTAGE_TOKENS = 512;                                  // gathered tokens whose V rows are staged in shared memory
constexpr size_t ATT_DYN_SMEM = (size_t)VSTAGE_TOKENS * (D + 4);    // V codes [512][128] then V scales [512]

// grid (B * Hq), one 512-thread CTA per (sequence, query head), two CTAs per SM.
// The kernel is a chain of dependent steps (select -> page lookup -> K gather -> softmax -> V gather), so what it costs
// is the number of memory round trips.  They are cut to three: (1) the block scores, selected with shuffle-based
// arg-max extraction when top_k <= 32 (no histogram passes); (2) the page ids of the gathered tokens; (3) ALL K rows
// in one batch of 16-byte loads (8 lanes per row, 64 rows per pass, 8 passes in flight) while the V rows and V scales
// of the same tokens travel to shared memory as per-thread asynchronous copies issued before the K loads -- by the
// time the softmax weights exist the V rows are already on chip.
// FUSED: the kernel also scores the blocks itself, and no scoring kernel runs before it.  It is launched in clusters of
// G CTAs -- the query heads of one kv-head, cluster rank = head within the group.  CTA r streams the 64-block tiles
// r, r + G, ... of the row's metadata (TMA into a two-stage ring that lies where the V rows are staged later), scores
// each tile for ALL heads of the group on the tensor cores exactly like quest_scores_mma_kernel, and PUSHES every head's
// scores into that head's CTA (stores into distributed shared memory, into the array that later holds the token
// weights).  After one cluster barrier every CTA has the scores of its own head in its shared memory: the score round
// trip through global memory, one launch and the wait between the two kernels are gone.  nb <= MAX_SEL_TOKENS.
template <int KVT, bool FUSED>
__global__ void __launch_bounds__(ATT_THREADS, 2)
quest_select_attend_kernel(const __grid_constant__ CUtensorMap tmM, const AttendParams p) {
    extern __shared__ __align__(16) uint8_t vstage[];   // ATT_DYN_SMEM bytes
    __shared__ __align__(16) uint32_t tk[TopkSmem<ATT_THREADS>::WORDS];
    __shared__ int sel[MAX_TOPK];
    __shared__ float w[MAX_SEL_TOKENS];
    __shared__ int2 where[MAX_SEL_TOKENS];  // (page, slot) of every gathered token; PAST_END set in slot past the sequence end
    __shared__ float qs[D];
    __shared__ float red[ATT_THREADS / 32];
    __shared__ float bcast[2];
    constexpr int NWARP = ATT_THREADS / 32, GROUPS = ATT_THREADS / 8;
    static_assert(MAX_SEL_TOKENS >= NWARP * D, "the weight array is reused for the per-warp partial outputs");

    const int row = blockIdx.x, hq = row % p.Hq, b = row / p.Hq, h = hq / p.G;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // q, seq_lens and the page table are older than the scoring kernel this launch depends on: read them first
    const int len = p.seq_lens ? min(max(p.seq_lens[b], 0), p.N) : p.N;
    const int nb = (len + p.block_size - 1) / p.block_size;  // blocks this sequence really has
    SKV_PHASE(0);
    for (int i = tid; i < D; i += ATT_THREADS) qs[i] = __half2float(p.q[(long long)row * D + i]);
    const float* sc = p.scores + (long long)row * p.nb;
    if (FUSED) {
        __shared__ __align__(8) unsigned long long fbar[4];   // full[2], empty[2]
        constexpr int FS = 2;                                  // ring stages of MS_STAGE_BYTES
        const uint32_t ring = (smem_u32(vstage) + 1023u) & ~1023u;
        const uint32_t full_bar = smem_u32(&fbar[0]), empty_bar = smem_u32(&fbar[2]);
        const int G = p.G, crank = (int)cluster_cta_rank();
        const int rowh = row / G;                              // (b, kv-head)
        const int tiles = (p.nb + MS_TILE - 1) / MS_TILE;
        const int my_tiles = crank < tiles ? (tiles - crank + G - 1) / G : 0;
        if (tid == 0) {
            for (int st = 0; st < FS; ++st) {
                mbar_init(full_bar + st * 8, 1);
                mbar_init(empty_bar + st * 8, MS_CONSUMER_WARPS);
            }
            fence_barrier_init();
        }
        __syncthreads();
        if (warp == MS_CONSUMER_WARPS) {            // producer: one lane, four boxes per tile
            if (lane == 0) {
                tma_prefetch_desc(&tmM);
                const uint64_t policy = l2_policy_evict_first();
                int st = 0;
                uint32_t ph = 0;
                for (int i = 0; i < my_tiles; ++i) {
                    if (i >= FS && !mbar_wait(empty_bar + st * 8, ph ^ 1u)) {
                        atomicOr(p.status, SKV_DEV_TIMEOUT);
                        break;
                    }
                    const uint32_t dst = ring + st * MS_STAGE_BYTES, bar = full_bar + st * 8;
                    mbar_expect_tx(bar, MS_STAGE_BYTES);
                    const int first = rowh * p.nb + (crank + i * G) * MS_TILE;
#pragma unroll
                    for (int hf = 0; hf < 4; ++hf) tma_load_2d(dst + hf * MS_BOX_BYTES, &tmM, bar, hf * 64, first, policy);
                    if (++st == FS) { st = 0; ph ^= 1u; }
                }
            }
        } else if (warp < MS_CONSUMER_WARPS) {      // consumers: warp w scores blocks 16w .. 16w+15 of every tile
            const int g = lane >> 2, tq = lane & 3, lj = lane >> 3, r8 = lane & 7;
            const uint32_t a_row_off = (uint32_t)((warp * 16 + (lj & 1) * 8 + r8) * 128);
            uint32_t qb[16][2];
            {
                const __half* qrow = p.q + ((long long)rowh * G + g) * D;
                const __half2 zero = __float2half2_rn(0.f);
#pragma unroll
                for (int kk2 = 0; kk2 < 8; ++kk2) {
                    __half2 u = zero, v = zero;
                    if (g < G) {
                        u = *reinterpret_cast<const __half2*>(qrow + kk2 * 16 + tq * 2);
                        v = *reinterpret_cast<const __half2*>(qrow + kk2 * 16 + 8 + tq * 2);
                    }
                    const __half2 un = __hmin2(u, zero), vn = __hmin2(v, zero), up = __hmax2(u, zero), vp = __hmax2(v, zero);
                    qb[kk2][0] = *reinterpret_cast<const uint32_t*>(&un);
                    qb[kk2][1] = *reinterpret_cast<const uint32_t*>(&vn);
                    qb[kk2 + 8][0] = *reinterpret_cast<const uint32_t*>(&up);
                    qb[kk2 + 8][1] = *reinterpret_cast<const uint32_t*>(&vp);
                }
            }
            // head 2tq lives in CTA 2tq of the cluster, head 2tq+1 in CTA 2tq+1: where this lane's results go
            const uint32_t w_local = smem_u32(w);
            const uint32_t dst0 = 2 * tq < G ? cluster_map(w_local, 2 * tq) : 0u;
            const uint32_t dst1 = 2 * tq + 1 < G ? cluster_map(w_local, 2 * tq + 1) : 0u;
            int st = 0;
            uint32_t ph = 0;
            for (int i = 0; i < my_tiles; ++i) {
                int ok = 1;
                if (lane == 0) ok = mbar_wait(full_bar + st * 8, ph) ? 1 : 0;
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) {
                    if (lane == 0) atomicOr(p.status, SKV_DEV_TIMEOUT);
                    break;
                }
                const uint32_t base = ring + st * MS_STAGE_BYTES + a_row_off;
                float acc0[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int kk2 = 0; kk2 < 16; ++kk2) {
                    const int c = 2 * kk2 + (lj >> 1);
                    uint32_t a[4];
                    ldsm_x4(base + (uint32_t)(c >> 3) * MS_BOX_BYTES + (uint32_t)(((c & 7) ^ r8) << 4), a[0], a[1], a[2], a[3]);
                    if (kk2 & 1) mma_f16(acc1, a, qb[kk2][0], qb[kk2][1]);
                    else mma_f16(acc0, a, qb[kk2][0], qb[kk2][1]);
                }
                const int j = (crank + i * G) * MS_TILE + warp * 16 + g;
                if (dst0) {
                    if (j < p.nb) st_cluster_f32(dst0 + j * 4, (acc0[0] + acc1[0]) * p.scale);
                    if (j + 8 < p.nb) st_cluster_f32(dst0 + (j + 8) * 4, (acc0[2] + acc1[2]) * p.scale);
                }
                if (dst1) {
                    if (j < p.nb) st_cluster_f32(dst1 + j * 4, (acc0[1] + acc1[1]) * p.scale);
                    if (j + 8 < p.nb) st_cluster_f32(dst1 + (j + 8) * 4, (acc0[3] + acc1[3]) * p.scale);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty_bar + st * 8);
                if (++st == FS) { st = 0; ph ^= 1u; }
            }
        }
        __syncwarp();
        cluster_barrier();    // every head's scores have arrived in its CTA (and every CTA is done with its ring)
        sc = w;
    } else {
        pdl_wait_prior_grids();   // launched as a programmatic dependent of the scoring kernel: its results are complete from here on
    }
    SKV_PHASE(1);
    const int kk = min(p.top_k, nb);
    if (kk <= 32 && nb <= ATT_THREADS * 4) block_topk_small<ATT_THREADS, 4>(sc, nb, kk, sel, reinterpret_cast<unsigned long long*>(tk));
    else if (kk <= 32 && nb <= ATT_THREADS * 16) block_topk_small<ATT_THREADS, 16>(sc, nb, kk, sel, reinterpret_cast<unsigned long long*>(tk));
    else block_topk_sorted_auto<ATT_THREADS, 16>(sc, nb, kk, sel, tk);
    __syncthreads();
    if (p.block_idx)
        for (int i = tid; i < p.top_k; i += ATT_THREADS) p.block_idx[(long long)row * p.top_k + i] = i < kk ? sel[i] : -1;

    SKV_PHASE(2);
    const int sub = tid & 7, grp = tid >> 3;  // 8 lanes per token row; grp in [0, 64)
    const int ntok = kk * p.block_size;
    const bool staged = ntok <= VSTAGE_TOKENS;
    float* vsc_sm = reinterpret_cast<float*>(vstage + (size_t)VSTAGE_TOKENS * D);
    // resolve every gathered token's page once (one page-table read per token, all in flight together)
    bool bad_page = false;
    for (int r = tid; r < ntok; r += ATT_THREADS) {
        const int t = SKV_INDEX(sel[r / p.block_size], p.nb) * p.block_size + r % p.block_size;
        // a token past the end points at the last real token and carries a flag, so that every later load has a
        // valid address and needs no condition (conditional loads are issued one behind the other)
        const int tc = min(t, len - 1);
        const int pg = checked_page(phys_page(p.page_table, b, p.max_pages, SKV_INDEX(tc / p.page_size, p.max_pages)), p.num_pages, bad_page);
        const int slot = tc % p.page_size;
        where[r] = make_int2(pg, slot | (t < len ? 0 : PAST_END));
        if (staged) cp_async4(smem_u32(vsc_sm + r), p.v.scales + pg * p.v.csp + h * p.v.csh + slot);
    }
    __syncthreads();

    SKV_PHASE(3);
    // ---- scores of the gathered tokens: 8 lanes per token row, 64 rows per pass
    float qv[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) qv[i] = qs[sub * 16 + i];
    constexpr int RU = 8;  // token rows per group and step: their code and scale loads are issued back to back
    float mx = -INFINITY;
    for (int r0 = 0; r0 < ntok; r0 += RU * GROUPS) {  // uniform trip count: the shuffles need whole warps
        uint4 raw[RU];
        float ksc[RU];
#pragma unroll
        for (int u = 0; u < RU; ++u) {
            const int2 pw = where[min(r0 + u * GROUPS + grp, ntok - 1)];
            const int slot = pw.y & ~PAST_END;
            raw[u] = ld_stream16(p.k.codes + pw.x * p.k.sp + h * p.k.sh + slot * p.k.ss + sub * 16);
            ksc[u] = __ldg(p.k.scales + pw.x * p.k.csp + h * p.k.csh + slot);
        }
        if (staged && r0 == 0) {
            // V rows on their way to shared memory (8 x 16 bytes per row, nothing held in registers), queued BEHIND
            // the K loads above: K is needed first, V only after the softmax.
            const uint32_t vdst = smem_u32(vstage);
            const int cshift = p.v4 ? 2 : 3;   // 16-byte chunks per V row: 4 (4-bit codes) or 8
            for (int c = tid; c < (ntok << cshift); c += ATT_THREADS) {
                const int2 pw = where[c >> cshift];
                cp_async16(vdst + c * 16, p.v.codes + pw.x * p.v.sp + h * p.v.sh + (pw.y & ~PAST_END) * p.v.ss +
                                              (c & ((1 << cshift) - 1)) * 16);
            }
        }
#pragma unroll
        for (int u = 0; u < RU; ++u) {
            const int r = r0 + u * GROUPS + grp;
            const bool valid = r < ntok && !(where[min(r, ntok - 1)].y & PAST_END);
            float x[16];
            unpack16<KVT>(raw[u], x);
            float d = 0.f;
#pragma unroll
            for (int i = 0; i < 16; ++i) d = fmaf(x[i], qv[i], d);
            d += __shfl_xor_sync(0xffffffffu, d, 1);
            d += __shfl_xor_sync(0xffffffffu, d, 2);
            d += __shfl_xor_sync(0xffffffffu, d, 4);
            const float sv = valid ? d * ksc[u] * p.scale : -INFINITY;
            if (sub == 0 && r < ntok) w[r] = sv;
            mx = fmaxf(mx, sv);
        }
    }
    SKV_PHASE(4);
    mx = warp_max(mx);
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    if (warp == 0) {
        float m2 = lane < NWARP ? red[lane] : -INFINITY;
        m2 = warp_max(m2);
        if (lane == 0) bcast[0] = m2;
    }
    __syncthreads();
    mx = bcast[0];
    float sum = 0.f;
    for (int r = tid; r < ntok; r += ATT_THREADS) {
        const float e = w[r] == -INFINITY ? 0.f : __expf(w[r] - mx);
        w[r] = e;
        sum += e;
    }
    sum = warp_sum(sum);
    if (lane == 0) red[warp] = sum;
    if (staged) cp_async_wait_all();   // this thread's V copies have landed; the barrier below publishes everybody's
    __syncthreads();
    if (warp == 0) {
        float s2 = lane < NWARP ? red[lane] : 0.f;
        s2 = warp_sum(s2);
        if (lane == 0) bcast[1] = s2;
    }
    __syncthreads();
    const float inv = bcast[1] > 0.f ? 1.f / bcast[1] : 0.f;

    SKV_PHASE(5);
    // ---- out = sum_t p_t * vs_t * vc_t
    float acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.f;
    if (staged) {
        // the weight of a token past the end is an exact zero and its row is a real (clamped) one, so no flag test
        for (int r = grp; r < ntok; r += GROUPS) {
            const float wt = w[r] * vsc_sm[r];
            float x[16];
            if (p.v4) unpack16_v4(*reinterpret_cast<const uint2*>(vstage + (size_t)r * (D / 2) + sub * 8), x);
            else unpack16<KVT>(*reinterpret_cast<const uint4*>(vstage + (size_t)r * D + sub * 16), x);
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[i] = fmaf(wt, x[i], acc[i]);
        }
    } else {
        for (int r0 = grp; r0 < ntok; r0 += RU * GROUPS) {
            uint4 raw[RU];
            float wt[RU];
#pragma unroll
            for (int u = 0; u < RU; ++u) {
                const int r = r0 + u * GROUPS;
                const int2 pw = where[min(r, ntok - 1)];
                const int slot = pw.y & ~PAST_END;
                raw[u] = ld_stream16(p.v.codes + pw.x * p.v.sp + h * p.v.sh + slot * p.v.ss + sub * 16);
                // the weight of a token past the end is already an exact zero; rows past ntok get zero here
                const float vs = __ldg(p.v.scales + pw.x * p.v.csp + h * p.v.csh + slot);
                wt[u] = r < ntok ? w[min(r, ntok - 1)] * vs : 0.f;
            }
#pragma unroll
            for (int u = 0; u < RU; ++u) {
                float x[16];
                unpack16<KVT>(raw[u], x);
#pragma unroll
                for (int i = 0; i < 16; ++i) acc[i] = fmaf(wt[u], x[i], acc[i]);
            }
        }
    }
    SKV_PHASE(6);
    // reduce the 64 row-groups: first inside each warp (4 groups), then across the warps through shared memory
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], 8);
        acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], 16);
    }
    __syncthreads();
    float* part = w;  // the token weights are no longer needed: reuse as [NWARP][D]
    if (lane < 8) {
#pragma unroll
        for (int i = 0; i < 16; ++i) part[warp * D + sub * 16 + i] = acc[i];
    }
    __syncthreads();
    for (int d = tid; d < D; d += ATT_THREADS) {
        float o = 0.f;
#pragma unroll
        for (int w2 = 0; w2 < NWARP; ++w2) o += part[w2 * D + d];
        p.out[(long long)row * D + d] = __float2half_rn(o * inv);
    }
    report_bad_page(bad_page, p.status);
    SKV_PHASE(7);
    SKV_PHASE_LAST_END();
}

}  // namespace quest
}  // namespace skv

using namespace skv;

static int check_pool_args(const void* codes, const float* scales, int page_size, long long ss, const char* what) {
    if (!codes || !scales) return fail(SKV_ERR_BAD_ARG, "%s: null pool pointer", what);
    if (page_size <= 0) return fail(SKV_ERR_BAD_ARG, "%s: page_size must be positive", what);
    if (reinterpret_cast<uintptr_t>(codes) & 15) return fail(SKV_ERR_BAD_ARG, "%s: code pool must be 16-byte aligned", what);
    if (ss % 16) return fail(SKV_ERR_BAD_ARG, "%s: slot stride must be a multiple of 16 bytes", what);
    return SKV_OK;
}

extern "C" {

#ifdef SKV_PROFILE_PHASES
int skv_debug_phase_ts_quest(unsigned long long* out) {
    return cudaMemcpyFromSymbol(out, skv_phase_ts, sizeof(unsigned long long) * 32) == cudaSuccess ? 0 : -4;
}
#endif

// 1: where it applies (tensor-core scoring on, up to 8 heads per group, at most 2048 blocks per sequence) ONE kernel
// scores the blocks and attends: clusters of G CTAs share a kv-head's metadata and exchange the scores through
// distributed shared memory; 0 (default): the scoring kernel followed by the select/attend kernel.  The two measure
// the same on B200 -- the fused scoring phase streams at the full HBM rate (10.5 us for 67 MB), but the two-kernel path
// hides the second launch and its prologue behind the scoring kernel.  Process-wide.
int skv_quest_set_fused(int on) {
    quest::fused_flag() = on ? 1 : 0;
    return SKV_OK;
}

// 1 (default): the block scores are computed by the tensor-core kernel that streams the metadata through a
// shared-memory ring (up to 8 query heads per kv-head; larger groups always use the other kernel); 0: by the
// register-load kernel.  The two sum the same exact products in different
// orders (fp32), so scores agree to rounding.
int skv_quest_set_ring_scores(int on) {
    quest::ring_scores_flag() = on ? 1 : 0;
    return SKV_OK;
}

// Number of metadata blocks for a cache of N tokens.
int skv_quest_num_blocks(int N, int block_size) { return (N <= 0 || block_size <= 0) ? 0 : (N + block_size - 1) / block_size; }

size_t skv_quest_workspace_bytes(int B, int Hq, int N, int block_size) {
    const int nb = skv_quest_num_blocks(N, block_size);
    if (B <= 0 || Hq <= 0 || nb <= 0) return 0;
    return 256 + (((size_t)B * Hq * nb * sizeof(float) + 255) & ~size_t(255));
}

int skv_quest_build_meta(const void* k_pool, const float* k_scale_pool, const int* page_table, const int* seq_lens,
                         void* meta_out, int B, int N, int Hkv, int D, int kv_dtype, int block_size, int page_size,
                         int max_pages, int num_pages, long long pool_stride_page, long long pool_stride_head,
                         long long pool_stride_slot, long long scale_stride_page, long long scale_stride_head,
                         int* status, int device, void* stream) {
    if (!meta_out) return fail(SKV_ERR_BAD_ARG, "skv_quest_build_meta: null output");
    int rc = check_pool_args(k_pool, k_scale_pool, page_size, pool_stride_slot, "skv_quest_build_meta");
    if (rc) return rc;
    if (B <= 0 || N <= 0 || Hkv <= 0 || block_size <= 0 || max_pages <= 0 || num_pages <= 0)
        return fail(SKV_ERR_BAD_ARG, "skv_quest_build_meta: sizes must be positive");
    if (D != quest::D) return fail(SKV_ERR_UNSUPPORTED, "head dim %d not supported (128)", D);
    if (kv_dtype != SKV_KV_I8 && kv_dtype != SKV_KV_E4M3) return fail(SKV_ERR_UNSUPPORTED, "kv_dtype %d is not an 8-bit type", kv_dtype);
    if ((long long)max_pages * page_size < N) return fail(SKV_ERR_BAD_ARG, "max_pages * page_size < N");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(SKV_ERR_CUDA, "cannot switch to device %d", device);
    quest::MetaParams p;
    p.k.codes = static_cast<const uint8_t*>(k_pool); p.k.scales = k_scale_pool;
    p.k.sp = pool_stride_page; p.k.sh = pool_stride_head; p.k.ss = pool_stride_slot;
    p.k.csp = scale_stride_page; p.k.csh = scale_stride_head;
    p.page_table = page_table; p.seq_lens = seq_lens; p.meta = static_cast<__half*>(meta_out);
    p.B = B; p.Hkv = Hkv; p.N = N; p.nb = skv_quest_num_blocks(N, block_size);
    p.block_size = block_size; p.page_size = page_size; p.max_pages = max_pages;
    p.num_pages = num_pages; p.status = status;
    const long long items = (long long)B * Hkv * p.nb;
    long long blocks = (items + quest::META_THREADS / 32 - 1) / (quest::META_THREADS / 32);
    const long long cap = (long long)sm_count(device) * 16;
    if (blocks > cap) blocks = cap;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (kv_dtype == SKV_KV_E4M3) quest::block_meta_build_kernel<SKV_KV_E4M3><<<(unsigned)blocks, quest::META_THREADS, 0, st>>>(p);
    else quest::block_meta_build_kernel<SKV_KV_I8><<<(unsigned)blocks, quest::META_THREADS, 0, st>>>(p);
    SKV_CUDA_TRY(cudaGetLastError());
    return SKV_OK;
}

int skv_quest_decode(const void* q, const void* k_pool, const void* v_pool, const float* k_scale_pool,
                     const float* v_scale_pool, const int* page_table, const int* seq_lens, const void* meta,
                     void* out, int* block_idx_out, void* workspace, size_t workspace_bytes, int B, int N, int Hq,
                     int Hkv, int D, int kv_dtype, int block_size, int top_k_blocks, int page_size, int max_pages,
                     int num_pages, long long pool_stride_page, long long pool_stride_head, long long pool_stride_slot,
                     long long scale_stride_page, long long scale_stride_head, float scale, int device, void* stream) {
    if (!q || !meta || !out) return fail(SKV_ERR_BAD_ARG, "skv_quest_decode: null tensor pointer");
    int rc = check_pool_args(k_pool, k_scale_pool, page_size, pool_stride_slot, "skv_quest_decode");
    if (rc) return rc;
    rc = check_pool_args(v_pool, v_scale_pool, page_size, pool_stride_slot, "skv_quest_decode");
    if (rc) return rc;
    if (B <= 0 || N <= 0 || Hq <= 0 || Hkv <= 0 || max_pages <= 0 || num_pages <= 0)
        return fail(SKV_ERR_BAD_ARG, "skv_quest_decode: sizes must be positive");
    if (Hq % Hkv != 0) return fail(SKV_ERR_BAD_ARG, "Hq=%d must be divisible by Hkv=%d", Hq, Hkv);
    const int G = Hq / Hkv;
    if (G > 8) return fail(SKV_ERR_UNSUPPORTED, "group size %d exceeds 8", G);
    if (D != quest::D) return fail(SKV_ERR_UNSUPPORTED, "head dim %d not supported (128)", D);
    const int v4 = (kv_dtype & SKV_V_INT4) ? 1 : 0;   // mixed-precision page records: V in 4 bits, 64 bytes per token
    kv_dtype &= ~SKV_V_INT4;
    if (kv_dtype != SKV_KV_I8 && kv_dtype != SKV_KV_E4M3) return fail(SKV_ERR_UNSUPPORTED, "kv_dtype %d is not an 8-bit type", kv_dtype);
    if (block_size <= 0 || top_k_blocks <= 0) return fail(SKV_ERR_BAD_ARG, "block_size and top_k_blocks must be positive");
    if (v4 && (long long)top_k_blocks * block_size > quest::VSTAGE_TOKENS)
        return fail(SKV_ERR_UNSUPPORTED, "with 4-bit values top_k_blocks * block_size must not exceed %d tokens", quest::VSTAGE_TOKENS);
    if (top_k_blocks > quest::MAX_TOPK || (long long)top_k_blocks * block_size > quest::MAX_SEL_TOKENS)
        return fail(SKV_ERR_UNSUPPORTED, "top_k_blocks * block_size = %lld exceeds %d tokens (or %d blocks)",
                    (long long)top_k_blocks * block_size, quest::MAX_SEL_TOKENS, quest::MAX_TOPK);
    if ((long long)max_pages * page_size < N) return fail(SKV_ERR_BAD_ARG, "max_pages * page_size < N");
    if (Hkv > 65535 || B > 65535) return fail(SKV_ERR_UNSUPPORTED, "grid dimension too large");
    const size_t need = skv_quest_workspace_bytes(B, Hq, N, block_size);
    if (!workspace || workspace_bytes < need)
        return fail(SKV_ERR_WORKSPACE, "workspace of %zu bytes is smaller than the %zu required", workspace_bytes, need);
    DeviceGuard guard(device);
    if (!guard.ok) return fail(SKV_ERR_CUDA, "cannot switch to device %d", device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int nb = skv_quest_num_blocks(N, block_size);

    quest::ScoreParams sp;
    sp.q = static_cast<const __half*>(q);
    sp.meta = static_cast<const __half*>(meta);
    sp.scores = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + 256);
    sp.Hq = Hq; sp.Hkv = Hkv; sp.G = G; sp.nb = nb; sp.scale = scale;
    const long long rows = (long long)B * Hkv;
    const long long total_blocks = rows * nb;
    // One launch instead of two when the group's heads can share the scoring as a cluster: the attend kernel scores the
    // blocks itself (see its FUSED variant).  Needs the scores of a row to fit the token-weight array.
    static int cluster_ok[64][9] = {{0}};   // [device][G]: 0 unknown, 1 no, 2 yes
    bool fused = quest::fused_flag() && quest::use_ring_scores() && G <= 8 && nb <= quest::MAX_SEL_TOKENS && device < 64;
    CUtensorMap tmF;
    memset(&tmF, 0, sizeof(tmF));
    if (fused) {
        if (cluster_ok[device][G] == 0) {
            bool ok = cudaFuncSetAttribute(quest::quest_select_attend_kernel<SKV_KV_E4M3, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)quest::ATT_DYN_SMEM) == cudaSuccess &&
                      cudaFuncSetAttribute(quest::quest_select_attend_kernel<SKV_KV_I8, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)quest::ATT_DYN_SMEM) == cudaSuccess;
            ok = ok && max_active_clusters_x(quest::quest_select_attend_kernel<SKV_KV_E4M3, true>, dim3(quest::ATT_THREADS), quest::ATT_DYN_SMEM, G) > 0;
            cudaGetLastError();
            cluster_ok[device][G] = ok ? 2 : 1;
        }
        fused = cluster_ok[device][G] == 2;
    }
    if (fused) {
        const int mrc = make_matrix_tmap(&tmF, meta, total_blocks, 2 * quest::D, 2 * quest::D, quest::MS_TILE, 64, false);
        if (mrc) return mrc;
    } else if (quest::use_ring_scores() && G <= 8) {
        // tensor-core scoring: one persistent CTA per SM, each a contiguous range of (row, 64-block tile) items
        static bool ms_configured[64] = {false};
        if (device < 64 && !ms_configured[device]) {
            SKV_CUDA_TRY(cudaFuncSetAttribute(quest::quest_scores_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)quest::MS_SMEM));
            ms_configured[device] = true;
        }
        CUtensorMap tmM;
        const int mrc = make_matrix_tmap(&tmM, meta, total_blocks, 2 * quest::D, 2 * quest::D, quest::MS_TILE, 64, false);
        if (mrc) return mrc;
        const int tiles_per_row = (nb + quest::MS_TILE - 1) / quest::MS_TILE;
        const long long total_items = rows * tiles_per_row;
        int ctas = sm_count(device);
        const long long per = (total_items + ctas - 1) / ctas;
        ctas = (int)((total_items + per - 1) / per);
        int* st_word = reinterpret_cast<int*>(workspace);
        quest::quest_scores_mma_kernel<<<ctas, quest::MS_THREADS, quest::MS_SMEM, st>>>(tmM, sp, tiles_per_row, total_items, per, st_word);
        SKV_CUDA_TRY(cudaGetLastError());
    } else {
    // One wave of two CTAs per SM; every warp takes blocks_per_warp consecutive blocks of the flattened space.  U (loads
    // of each half in flight per lane) is picked so that the iterations cover the space with the smallest idle tail.
    int ctas = sm_count(device) * 2;
    const long long warps = (long long)ctas * (quest::SCORE_THREADS / 32);
    const long long share = (total_blocks + warps - 1) / warps;   // blocks a warp must take at least
    const int umax = G <= 4 ? 8 : 4, umin = G <= 4 ? 5 : 3;
    int best_u = umax;
    long long best_cover = -1;
    for (int u = umax; u >= umin; --u) {
        const long long per = (share + 2 * u - 1) / (2 * u) * (2 * u);
        if (best_cover < 0 || per < best_cover) { best_cover = per; best_u = u; }
    }
    const int blocks_per_warp = (int)best_cover;
    const long long need_ctas = (total_blocks + (long long)blocks_per_warp * 8 - 1) / ((long long)blocks_per_warp * 8);
    if (need_ctas < ctas) ctas = (int)need_ctas;
    cudaError_t le;
    if (G <= 4) {
        switch (best_u) {
            case 8: le = quest::launch_scores<4, 8>(sp, total_blocks, blocks_per_warp, ctas, st); break;
            case 7: le = quest::launch_scores<4, 7>(sp, total_blocks, blocks_per_warp, ctas, st); break;
            case 6: le = quest::launch_scores<4, 6>(sp, total_blocks, blocks_per_warp, ctas, st); break;
            default: le = quest::launch_scores<4, 5>(sp, total_blocks, blocks_per_warp, ctas, st); break;
        }
    } else {
        le = best_u == 4 ? quest::launch_scores<8, 4>(sp, total_blocks, blocks_per_warp, ctas, st)
                         : quest::launch_scores<8, 3>(sp, total_blocks, blocks_per_warp, ctas, st);
    }
    SKV_CUDA_TRY(le);

    }

    quest::AttendParams ap;
    ap.q = sp.q; ap.scores = sp.scores;
    ap.k.codes = static_cast<const uint8_t*>(k_pool); ap.k.scales = k_scale_pool;
    ap.v.codes = static_cast<const uint8_t*>(v_pool); ap.v.scales = v_scale_pool;
    ap.k.sp = ap.v.sp = pool_stride_page; ap.k.sh = ap.v.sh = pool_stride_head; ap.k.ss = ap.v.ss = pool_stride_slot;
    ap.k.csp = ap.v.csp = scale_stride_page; ap.k.csh = ap.v.csh = scale_stride_head;
    ap.page_table = page_table; ap.seq_lens = seq_lens;
    ap.out = static_cast<__half*>(out); ap.block_idx = block_idx_out;
    ap.Hq = Hq; ap.G = G; ap.N = N; ap.nb = nb; ap.block_size = block_size; ap.page_size = page_size;
    ap.max_pages = max_pages; ap.top_k = top_k_blocks; ap.scale = scale;
    ap.num_pages = num_pages;
    ap.v4 = v4;
    if (v4) ap.v.ss = quest::D / 2;
    ap.status = reinterpret_cast<int*>(workspace);   // status word at offset 0, as skv_workspace_status reads it
    static bool configured[64] = {false};
    if (device < 64 && !configured[device]) {
        SKV_CUDA_TRY(cudaFuncSetAttribute(quest::quest_select_attend_kernel<SKV_KV_E4M3, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)quest::ATT_DYN_SMEM));
        SKV_CUDA_TRY(cudaFuncSetAttribute(quest::quest_select_attend_kernel<SKV_KV_I8, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)quest::ATT_DYN_SMEM));
        configured[device] = true;
    }
    const dim3 agrid((unsigned)(B * Hq)), ablock(quest::ATT_THREADS);
    if (fused) {   // clusters of G CTAs along x: the query heads of one kv-head
        if (kv_dtype == SKV_KV_E4M3) SKV_CUDA_TRY(launch_cluster_x(quest::quest_select_attend_kernel<SKV_KV_E4M3, true>, agrid, ablock, quest::ATT_DYN_SMEM, st, G, tmF, ap));
        else SKV_CUDA_TRY(launch_cluster_x(quest::quest_select_attend_kernel<SKV_KV_I8, true>, agrid, ablock, quest::ATT_DYN_SMEM, st, G, tmF, ap));
    } else if (kv_dtype == SKV_KV_E4M3) {
        SKV_CUDA_TRY(launch_pdl(quest::quest_select_attend_kernel<SKV_KV_E4M3, false>, agrid, ablock, quest::ATT_DYN_SMEM, st, tmF, ap));
    } else {
        SKV_CUDA_TRY(launch_pdl(quest::quest_select_attend_kernel<SKV_KV_I8, false>, agrid, ablock, quest::ATT_DYN_SMEM, st, tmF, ap));
    }
    SKV_CUDA_TRY(cudaGetLastError());
    return SKV_OK;
}

}  // extern "C"

SKV_BOUNDS_GETTER(skv_debug_bounds_paged_quest)
