// Fused KV eviction: score-based token selection, compaction, and quantisation
// of the surviving rows to INT8 or FP8-E4M3 with per-token-per-head fp32 scales.
//
// The reference has no working CUDA implementation of this operation: its
// fused_kv_evict calls a binding with the wrong arity (sparse_kv/eviction.py:23-26
// against csrc/pybind/bindings.cpp:3-5) and its launcher rejects INT8
// (csrc/kernels/kv_evict_quant.cu:294).  The arithmetic followed here is the
// reference's PyTorch path _reference_eviction (sparse_kv/eviction.py:30-44):
// topk over the scores, gather of the chosen rows, optional int8 cast -- extended
// by scaled quantisation and an always-kept window of recent tokens.
//
// The evicted rows are never read.  Kernels:
//   evict_fused_cluster_kernel -- the single-pass path (position order, rows of up to 32 K competing scores, D = 64
//      or 128): a thread-block cluster of four 1024-thread CTAs per (b, h) keeps the row's score keys in registers,
//      finds the exact budget-th largest with four radix passes whose digit histograms are summed across the
//      cluster through distributed shared memory, writes the ascending position list, and then the same four CTAs
//      gather and quantise that head's surviving K and V rows, a quarter of the list each -- no second launch and
//      no wait for other heads.
//   evict_select_cluster_kernel / evict_select_kernel + evict_gather_quant_kernel -- the two-launch path for
//      everything else (descending-score order re-sorts with a shared-memory bitonic sort; longer rows take the
//      single-CTA radix select).
//   Quantisation: D/8 lanes per surviving row, 16-byte loads, row amax by shuffles, scale = amax / qmax by one IEEE
//      divide per row, codes by multiplication with the reciprocal and a magic-number round-half-even, with the
//      IEEE divide redone only where the product lies within 1e-4 of a rounding boundary (INT8 codes are bit-exact).
#include <cooperative_groups.h>
#include <cuda_fp8.h>

#include "skv_common.cuh"
#include "skv_select.cuh"

#define SKV_QUANT_NONE 0   // fp16 rows copied unchanged
#define SKV_QUANT_INT8 1   // symmetric int8, scale = amax / 127
#define SKV_QUANT_E4M3 2   // fp8 e4m3 (finite, max 448), scale = amax / 448
#define SKV_QUANT_CAST 3   // the reference's bare `.to(torch.int8)`: truncate toward zero, no scale

#define SKV_ORDER_POSITION 0
#define SKV_ORDER_SCORE 1

namespace skv {
namespace evq {

constexpr int SEL_THREADS = 1024;
constexpr int MAX_KEEP = 8192;
constexpr int GQ_THREADS = 256;

struct SelectParams {
    const float* scores;  // [rows, T]
    int* idx;             // [rows, keep]
    int T, budget, recent, keep, order;
};

__global__ void __launch_bounds__(SEL_THREADS)
evict_select_kernel(const SelectParams p) {
    pdl_launch_dependents();  // the kernel that consumes the kept positions may be scheduled now; it waits for this grid to finish
    extern __shared__ uint32_t dsm[];
    uint32_t* tk = dsm;
    int* sel = reinterpret_cast<int*>(tk + TopkSmem<SEL_THREADS>::WORDS);  // [pow2 >= keep]
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* sc = p.scores + (long long)row * p.T;
    const int recent = min(p.recent, p.T);
    const int head = p.T - recent;              // positions competing on score
    const int kb = min(p.budget, head);         // how many of them survive
    block_topk_sorted_auto<SEL_THREADS, 16>(sc, head, kb, sel, tk);
    for (int i = tid; i < recent; i += SEL_THREADS) sel[kb + i] = head + i;
    __syncthreads();
    const int keep = kb + recent;  // equals p.keep by construction on the host
    int* out = p.idx + (long long)row * p.keep;
    if (p.order == SKV_ORDER_POSITION) {
        for (int i = tid; i < keep; i += SEL_THREADS) out[i] = sel[i];
        return;
    }
    // descending score, lower position first among equals: bitonic sort of (key, position)
    int n2 = 1;
    while (n2 < keep) n2 <<= 1;
    uint32_t* key = reinterpret_cast<uint32_t*>(sel + MAX_KEEP);
    for (int i = tid; i < n2; i += SEL_THREADS) {
        if (i < keep) {
            key[i] = ~score_key(sc[sel[i]]);  // ascending ~key == descending score
        } else {
            key[i] = 0xFFFFFFFFu;
            sel[i] = 0x7FFFFFFF;
        }
    }
    __syncthreads();
    for (int size = 2; size <= n2; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int t = tid; t < n2 / 2; t += SEL_THREADS) {
                const int lo = 2 * t - (t & (stride - 1));  // index with the `stride` bit clear
                const int hi = lo + stride;
                const bool up = (lo & size) == 0;
                const uint32_t ka = key[lo], kb2 = key[hi];
                const int ia = sel[lo], ib = sel[hi];
                const bool a_after_b = ka > kb2 || (ka == kb2 && ia > ib);
                if (a_after_b == up) {
                    key[lo] = kb2; key[hi] = ka;
                    sel[lo] = ib; sel[hi] = ia;
                }
            }
            __syncthreads();
        }
    }
    for (int i = tid; i < keep; i += SEL_THREADS) out[i] = sel[i];
}

// ---------------------------------------------------------------------------
// Cluster variant of the selection (position order only).  One CTA is issue-bound at about 6 us per radix
// pass over 32 K scores, so a thread-block cluster of CL CTAs shares each (b, h) row: every CTA keeps its
// slice of the keys in registers (loaded once), the per-pass digit histograms are summed across the cluster
// through distributed shared memory, and each CTA writes its part of the ascending position list.
// Serves rows of up to CL * 1024 * KR competing scores; longer rows take the single-CTA kernel.
// ---------------------------------------------------------------------------
constexpr int CL = 4;   // CTAs per cluster
constexpr int KR = 8;   // keys per thread

constexpr int MAX_CAND = 1024;   // threshold-bucket size up to which the last 16 key bits are resolved by ranking

// Exact top-`budget` of one (b, h) row by a cluster of CL CTAs; writes the ascending position list.
// Whatever CTAs exchange is PUSHED: the owner stores its counts into every CTA's shared memory before the cluster
// barrier, so that after the barrier everything is local (a remote load costs a round trip of about a microsecond on
// the critical path, a remote store costs nothing the barrier does not already wait for).
// Two 8-bit radix passes fix the upper 16 key bits.  The bucket that holds the budget-th key is then usually a few
// hundred keys: its members are pushed to every CTA (key, then complemented position: among equal scores the lower
// position ranks higher) and each member counts how many members outrank it; the one outranked by exactly
// remaining - 1 others is the last key kept.  Larger buckets (many equal scores) take two more radix passes.
__device__ __forceinline__ void cluster_select_row(const SelectParams& p, cooperative_groups::cluster_group& cluster) {
    constexpr int NW = SEL_THREADS / 32;
    static_assert(NW == 32, "warp 0 scans one count per warp with its 32 lanes");
    __shared__ uint32_t hist[NW * 256];        // per-warp private digit counts; later the candidate list
    __shared__ uint32_t xhist[2][CL][256];     // every CTA's folded counts of a pass (pushed), double-buffered across passes
    __shared__ uint32_t thist[256];            // cluster-wide counts
    __shared__ uint32_t wcnt[4 * NW];
    __shared__ uint32_t xtot[CL][2];           // every CTA's (greater, equal) totals (pushed)
    __shared__ uint32_t bc[6];                 // digit, remaining, bucket size; threshold key and tie count of the ranking step
    __shared__ uint32_t ncand;                 // CTA 0's copy hands out slots of the candidate list

    SKV_PHASE(0);
    const int crank = (int)cluster.block_rank();
    const int row = blockIdx.x / CL;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const float* sc = p.scores + (long long)row * p.T;
    const int recent = min(p.recent, p.T);
    const int head = p.T - recent;        // positions competing on score
    const int kb = min(p.budget, head);   // how many of them survive
    int* out = p.idx + (long long)row * p.keep;
    if (tid == 0) ncand = 0;              // two cluster barriers pass before anybody adds to it

    // slice of this CTA, then a contiguous 32-aligned segment per warp; lane l holds elements s0 + 32 j + l
    int span = (head + CL - 1) / CL;
    span = (span + 31) & ~31;
    const int e0 = min(head, crank * span), e1 = min(head, e0 + span);
    int seg = (span + NW - 1) / NW;
    seg = (seg + 31) & ~31;               // <= 32 * KR by the host-side size check
    const int s0 = min(e1, e0 + warp * seg), s1 = min(e1, s0 + seg);
    uint32_t key[KR];
    uint32_t have = 0;                    // bit j: element j exists
    {
        float raw[KR];   // unconditional loads at clamped positions: all in flight together
#pragma unroll
        for (int j = 0; j < KR; ++j) raw[j] = sc[min(s0 + j * 32 + lane, p.T - 1)];
#pragma unroll
        for (int j = 0; j < KR; ++j) {
            const int i = s0 + j * 32 + lane;
            key[j] = 0u;
            if (i < s1) { key[j] = score_key(raw[j]); have |= 1u << j; }
        }
    }

    SKV_PHASE(1);
    uint32_t thr = 0;
    int need = 0;
    if (kb < head && kb > 0) {
        uint32_t prefix = 0, mask = 0;
        int remaining = kb;
#pragma unroll 1
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            for (int i = tid; i < NW * 256; i += SEL_THREADS) hist[i] = 0;
            __syncthreads();
            uint32_t* myh = hist + warp * 256;
#pragma unroll
            for (int j = 0; j < KR; ++j) {
                const bool act = ((have >> j) & 1u) && (key[j] & mask) == prefix;
                const uint32_t digit = (key[j] >> shift) & 255u;
                const uint32_t voters = __ballot_sync(0xffffffffu, act);
                if (voters) {
                    const int leader = __ffs(voters) - 1;
                    const uint32_t d0 = __shfl_sync(0xffffffffu, digit, leader);
                    const uint32_t same = __ballot_sync(0xffffffffu, act && digit == d0);
                    if (same == voters) {
                        if (lane == leader) atomicAdd(&myh[d0], (uint32_t)__popc(voters));
                    } else if (act) {
                        atomicAdd(&myh[digit], 1u);
                    }
                }
            }
            __syncthreads();
            if (tid < 256) {
                uint32_t t = 0;
#pragma unroll 8
                for (int w = 0; w < NW; ++w) t += hist[w * 256 + tid];
#pragma unroll
                for (int c = 0; c < CL; ++c) cluster.map_shared_rank(&xhist[pass & 1][crank][0], c)[tid] = t;
            }
            cluster.sync();   // every CTA's folded counts of this pass have arrived here
            if (tid < 256) {
                uint32_t t = 0;
#pragma unroll
                for (int c = 0; c < CL; ++c) t += xhist[pass & 1][c][tid];
                thist[tid] = t;
            }
            __syncthreads();
            if (warp == 0) {  // same digit search as the single-CTA routine, on the cluster-wide counts
                uint32_t mine = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j) mine += thist[255 - 8 * lane - j];
                uint32_t incl = mine;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl += v;
                }
                const uint32_t hit = __ballot_sync(0xffffffffu, incl >= (uint32_t)remaining);
                const int owner = __ffs(hit) - 1;
                if (lane == owner) {
                    uint32_t above = incl - mine;
                    int d = 255 - 8 * lane;
                    for (int j = 0; j < 8; ++j, --d) {
                        const uint32_t c = thist[d];
                        if (above + c >= (uint32_t)remaining) break;
                        above += c;
                    }
                    bc[0] = (uint32_t)d;
                    bc[1] = (uint32_t)remaining - above;
                    bc[2] = thist[d];             // keys in the chosen bucket, cluster-wide
                }
            }
            __syncthreads();
            prefix |= bc[0] << shift;
            mask |= 0xFFu << shift;
            remaining = (int)bc[1];
            const uint32_t bucket = bc[2];
            SKV_PHASE(2 + pass);
            if (pass == 1 && bucket <= (uint32_t)MAX_CAND) {
                // hist is idle in every CTA by now (each finished its fold before the barrier above)
                unsigned long long* all64 = reinterpret_cast<unsigned long long*>(hist);   // [MAX_CAND], same content in every CTA
                uint32_t* slots = cluster.map_shared_rank(&ncand, 0);
#pragma unroll
                for (int j = 0; j < KR; ++j)
                    if (((have >> j) & 1u) && (key[j] & mask) == prefix) {
                        const uint32_t slot = atomicAdd(slots, 1u);
                        const unsigned long long me =
                            ((unsigned long long)key[j] << 32) | (0xFFFFFFFFu - (uint32_t)(s0 + j * 32 + lane));
#pragma unroll
                        for (int c = 0; c < CL; ++c) cluster.map_shared_rank(all64, c)[slot] = me;
                    }
                cluster.sync();
                const int n = (int)bucket;
                for (int i = tid; i < n; i += SEL_THREADS) {
                    const unsigned long long me = all64[i];
                    int rank = 0;
                    for (int q = 0; q < n; ++q) rank += all64[q] > me ? 1 : 0;
                    if (rank == remaining - 1) {
                        int ties = 0;   // members with the same key that are kept: this one and those ranked above it
                        for (int q = 0; q < n; ++q) ties += ((all64[q] >> 32) == (me >> 32) && all64[q] >= me) ? 1 : 0;
                        bc[3] = (uint32_t)(me >> 32);
                        bc[4] = (uint32_t)ties;
                    }
                }
                __syncthreads();
                prefix = bc[3];
                remaining = (int)bc[4];
                SKV_PHASE(6);
                break;
            }
            __syncthreads();   // bc is rewritten in the next pass
        }
        thr = prefix;
        need = remaining;
    } else {
        need = head;  // kb >= head: every competing score survives (thr = 0 makes every key "greater or equal")
    }

    SKV_PHASE(7);
    // per-warp counts of keys above / equal to the threshold
    uint32_t gt = 0, eq = 0;
#pragma unroll
    for (int j = 0; j < KR; ++j) {
        const bool in = (have >> j) & 1u;
        gt += __popc(__ballot_sync(0xffffffffu, in && (kb >= head || key[j] > thr)));
        eq += __popc(__ballot_sync(0xffffffffu, in && kb < head && key[j] == thr));
    }
    if (lane == 0) { wcnt[warp] = gt; wcnt[NW + warp] = eq; }
    __syncthreads();
    if (warp == 0) {   // this CTA's totals, pushed to everybody
        uint32_t g = wcnt[lane], e = wcnt[NW + lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            g += __shfl_xor_sync(0xffffffffu, g, o);
            e += __shfl_xor_sync(0xffffffffu, e, o);
        }
        if (lane < CL) {
            uint32_t* dst = cluster.map_shared_rank(&xtot[crank][0], lane);
            dst[0] = g;
            dst[1] = e;
        }
    }
    cluster.sync();
    // ties and selected positions in the CTAs before this one
    uint32_t eq_before = 0, sel_before = 0;
    for (int c = 0; c < crank; ++c) {
        const uint32_t g = xtot[c][0], e = xtot[c][1];
        sel_before += g + (uint32_t)max(0, min((int)e, need - (int)eq_before));
        eq_before += e;
    }
    if (warp == 0) {
        const uint32_t g = wcnt[lane], e = wcnt[NW + lane];   // NW == 32
        uint32_t ei = e;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t v = __shfl_up_sync(0xffffffffu, ei, o);
            if (lane >= o) ei += v;
        }
        const uint32_t eex = eq_before + ei - e;
        const uint32_t take = (uint32_t)max(0, min((int)e, need - (int)eex));
        const uint32_t sl = g + take;
        uint32_t si = sl;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t v = __shfl_up_sync(0xffffffffu, si, o);
            if (lane >= o) si += v;
        }
        wcnt[2 * NW + lane] = sel_before + si - sl;
        wcnt[3 * NW + lane] = eex;
    }
    __syncthreads();
    uint32_t pos = wcnt[2 * NW + warp], eqrun = wcnt[3 * NW + warp];
    const uint32_t lt = (1u << lane) - 1u;
    if (kb > 0) {
#pragma unroll
        for (int j = 0; j < KR; ++j) {
            const bool in = (have >> j) & 1u;
            const bool isgt = in && (kb >= head || key[j] > thr), iseq = in && kb < head && key[j] == thr;
            const uint32_t beq = __ballot_sync(0xffffffffu, iseq);
            const bool sel = isgt || (iseq && (int)(eqrun + __popc(beq & lt)) < need);
            const uint32_t bsel = __ballot_sync(0xffffffffu, sel);
            if (sel) out[SKV_INDEX(pos + __popc(bsel & lt), p.keep)] = s0 + j * 32 + lane;
            pos += __popc(bsel);
            eqrun += __popc(beq);
        }
    }
    if (crank == 0)
        for (int i = tid; i < recent; i += SEL_THREADS) out[kb + i] = head + i;
    SKV_PHASE(8);
    // Release/acquire at cluster scope: the position list written above is visible to the other CTAs of the cluster
    // after this barrier (the fused kernel reads it back), and nobody leaves while a neighbour may still write to or
    // read from its shared memory.
    cluster.sync();
    SKV_PHASE(9);
}

__global__ void __cluster_dims__(CL, 1, 1) __launch_bounds__(SEL_THREADS)
evict_select_cluster_kernel(const SelectParams p) {
    pdl_launch_dependents();  // the kernel that consumes the kept positions may be scheduled now; it waits for this grid to finish
    cooperative_groups::cluster_group cluster = cooperative_groups::this_cluster();
    cluster_select_row(p, cluster);
}

struct GatherParams {
    const __half* k;   // element (b,h,t,d) at b*sb + h*sh + t*st + d
    const __half* v;
    const int* idx;    // [rows, keep]
    void* k_out;       // [rows, keep, D]  fp16 or 1-byte codes
    void* v_out;
    float* k_scale;    // [rows, keep] (scaled modes only)
    float* v_scale;
    int H, keep, T;
    long long rows_total;  // B * H * keep
    long long sb, sh, st;
};

// a / b for a constant b, correctly rounded, in three instructions: with rb = RN(1/b) and q = RN(a * rb) (a faithful
// quotient), the residual r = a - q * b is exact in one FMA and RN(q + r * rb) is the correctly rounded a / b
// (Markstein's correction step; it holds for every b whose significand is not all ones -- 127 and 448 are not).
__device__ __forceinline__ float div_const_rn(float a, float b, float rb) {
    const float q = a * rb;
    const float r = fmaf(-q, b, a);
    return fmaf(r, rb, q);
}

// `valid` only guards the stores: every lane of the warp runs the shuffles.
// The quantisation is written for instruction count: with 8-bit outputs this code, not HBM, is what a gather of
// 256-byte rows costs.  Row maximum on packed halves (|x| and max are exact in fp16); one reciprocal per row; per
// element one FMA whose addend 1.5 * 2^23 rounds x * inv to the integer grid (half to even) and leaves the integer,
// in two's complement, in the low mantissa bits.  x * inv differs from the IEEE quotient x / scale by at most 2 ulp
// (<= 2e-5 for |q| <= 127), so the code can only differ where the product lies within 1e-4 of a rounding boundary:
// a second FMA forms that distance, one flag per lane collects "too close", and the rare lane with the flag set
// redoes its eight codes with the IEEE divide.  INT8 codes are therefore bit-exact; FP8 codes, allowed one code
// step, take the product as it is through the paired saturating conversion.
template <int MODE>
__device__ __forceinline__ void quant_row(const uint4& raw, int sub, int lpr, uint8_t* out_row, float* scale_out,
                                          __half* out_row_f16, bool valid) {
    if (MODE == SKV_QUANT_NONE) {
        if (valid) *reinterpret_cast<uint4*>(out_row_f16 + sub * 8) = raw;
        return;
    }
    const __half2* hx = reinterpret_cast<const __half2*>(&raw);
    float x[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(hx[i]);
        x[2 * i] = f.x;
        x[2 * i + 1] = f.y;
    }
    if (MODE == SKV_QUANT_CAST) {
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            lo |= (uint32_t)((int)x[i] & 0xFF) << (8 * i);      // cvt.rzi then wrap to 8 bits, as the host cast does
            hi |= (uint32_t)((int)x[4 + i] & 0xFF) << (8 * i);
        }
        if (valid) *reinterpret_cast<uint2*>(out_row + sub * 8) = make_uint2(lo, hi);
        return;
    }
    __half2 m2 = __hmax2(__hmax2(__habs2(hx[0]), __habs2(hx[1])), __hmax2(__habs2(hx[2]), __habs2(hx[3])));
    for (int o = lpr / 2; o > 0; o >>= 1) {
        const uint32_t t = __shfl_xor_sync(0xffffffffu, *reinterpret_cast<const uint32_t*>(&m2), o);
        m2 = __hmax2(m2, *reinterpret_cast<const __half2*>(&t));
    }
    const float amax = fmaxf(__low2float(m2), __high2float(m2));
    const float scale = amax > 0.f ? (MODE == SKV_QUANT_INT8 ? div_const_rn(amax, 127.f, 1.f / 127.f)
                                                             : div_const_rn(amax, 448.f, 1.f / 448.f))
                                   : 1.f;
    float inv;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(inv) : "f"(scale));   // within 1 ulp; the boundary test below covers it
    uint32_t lo, hi;
    if (MODE == SKV_QUANT_INT8) {
        constexpr float MAGIC = 12582912.f;
        // |x * inv| <= 127 (1 + 2^-22) because |x| <= amax = 127 * scale, so rounding already lands in [-127, 127]
        // Two reciprocals that bracket 1 / scale (the approximation is within 1 ulp, 1.2e-7 relative; they sit 3e-7 to
        // either side): x / scale, and its fp32 rounding, lie between x * inv_lo and x * inv_hi, so when both products
        // round to the same integer that integer is the code.  One xor-or per element collects "they differ".
        const float inv_lo = inv * (1.f - 3e-7f), inv_hi = inv * (1.f + 3e-7f);
        float r[8];
        uint32_t differ = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            r[i] = fmaf(x[i], inv_lo, MAGIC);
            differ |= __float_as_uint(r[i]) ^ __float_as_uint(fmaf(x[i], inv_hi, MAGIC));
        }
        if (differ) {
#pragma unroll
            for (int i = 0; i < 8; ++i) r[i] = __fdiv_rn(x[i], scale) + MAGIC;
        }
        // low bytes of eight words -> two words
        lo = __byte_perm(__byte_perm(__float_as_uint(r[0]), __float_as_uint(r[1]), 0x0040),
                         __byte_perm(__float_as_uint(r[2]), __float_as_uint(r[3]), 0x0040), 0x5410);
        hi = __byte_perm(__byte_perm(__float_as_uint(r[4]), __float_as_uint(r[5]), 0x0040),
                         __byte_perm(__float_as_uint(r[6]), __float_as_uint(r[7]), 0x0040), 0x5410);
    } else {
        uint32_t c[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
            c[i] = (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(x[2 * i] * inv, x[2 * i + 1] * inv), __NV_SATFINITE, __NV_E4M3);
        lo = __byte_perm(c[0], c[1], 0x5410);
        hi = __byte_perm(c[2], c[3], 0x5410);
    }
    if (valid) *reinterpret_cast<uint2*>(out_row + sub * 8) = make_uint2(lo, hi);
    if (valid && sub == 0) *scale_out = scale;
}

// Two-launch path: grid (chunks, B * H); one group of D/8 lanes per kept row, four rows per group and step, the CTAs
// of a (b, h) striding over its `keep` list entries.  No integer division anywhere on the row path.
#ifndef SKV_GATHER_MIN_CTAS
#define SKV_GATHER_MIN_CTAS 4
#endif
template <int D, int MODE>
__global__ void __launch_bounds__(GQ_THREADS, SKV_GATHER_MIN_CTAS)
evict_gather_quant_kernel(const GatherParams p) {
    pdl_wait_prior_grids();   // launched as a programmatic dependent of the selection kernel: its results are complete from here on
    constexpr int LPR = D / 8;
    constexpr int GPB = GQ_THREADS / LPR;
    constexpr int U = 4;
    const int sub = threadIdx.x % LPR, grp = threadIdx.x / LPR;
    const int row = blockIdx.y;                              // (b, h)
    const int b = row / p.H, h = row - b * p.H;
    const int* list = p.idx + (long long)row * p.keep;
    const long long base = (long long)b * p.sb + (long long)h * p.sh + sub * 8;
    const long long orow = (long long)row * p.keep;
    // Rows past the end repeat the list's last entry -- a real row that is in flight anyway -- and only their stores
    // are dropped: loads under a condition would be issued one by one, each behind the use of the one before.
    // The positions of the NEXT step are fetched while this step's rows are in flight, so a step costs one memory
    // round trip instead of two dependent ones.  The trip count is the same for every lane of a CTA.
    constexpr int CHUNK = GPB * U;
    const int step = gridDim.x * CHUNK;
    const int last = p.keep - 1;
    int tn[U];
#pragma unroll
    for (int u = 0; u < U; ++u) tn[u] = __ldg(list + min((int)blockIdx.x * CHUNK + u * GPB + grp, last));
    for (int jb = blockIdx.x * CHUNK; jb < p.keep; jb += step) {
        int t[U];
#pragma unroll
        for (int u = 0; u < U; ++u) t[u] = tn[u];
        if (jb + step < p.keep) {   // block-uniform
#pragma unroll
            for (int u = 0; u < U; ++u) tn[u] = __ldg(list + min(jb + step + u * GPB + grp, last));
        }
        uint4 kr[U], vr[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long long src = base + (long long)SKV_INDEX(max(t[u], 0), p.T) * p.st;
            kr[u] = ld_stream16(p.k + src);
            vr[u] = ld_stream16(p.v + src);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int j = jb + u * GPB + grp;
            const bool valid = j < p.keep;
            const long long r = orow + j;
            if (MODE == SKV_QUANT_NONE) {
                quant_row<MODE>(kr[u], sub, LPR, nullptr, nullptr, static_cast<__half*>(p.k_out) + r * D, valid);
                quant_row<MODE>(vr[u], sub, LPR, nullptr, nullptr, static_cast<__half*>(p.v_out) + r * D, valid);
            } else {
                quant_row<MODE>(kr[u], sub, LPR, static_cast<uint8_t*>(p.k_out) + r * D, p.k_scale + r, nullptr, valid);
                quant_row<MODE>(vr[u], sub, LPR, static_cast<uint8_t*>(p.v_out) + r * D, p.v_scale + r, nullptr, valid);
            }
        }
    }
}

// Selection and gather in one launch: after cluster_select_row the (b, h) row's ascending position list is complete
// in global memory (and in L2); CTA c of the cluster takes list entries [c * per, (c + 1) * per).  Same lane layout
// and quantisation as evict_gather_quant_kernel; U = 4 rows per lane group and step, the next step's positions
// fetched while this step's rows are in flight.
template <int D, int MODE>
__global__ void __cluster_dims__(CL, 1, 1) __launch_bounds__(SEL_THREADS)
evict_fused_cluster_kernel(const SelectParams p, const GatherParams g) {
    cooperative_groups::cluster_group cluster = cooperative_groups::this_cluster();
    cluster_select_row(p, cluster);

    constexpr int LPR = D / 8;
    constexpr int GPB = SEL_THREADS / LPR;
    constexpr int U = 4;
    const int crank = (int)cluster.block_rank();
    const long long row = blockIdx.x / CL;                 // (b, h)
    const int sub = threadIdx.x % LPR, grp = threadIdx.x / LPR;
    const int per = (p.keep + CL - 1) / CL;
    const int j0 = min(p.keep, crank * per), j1 = min(p.keep, j0 + per);
    if (j0 >= j1) return;
    SKV_PHASE(10);
    const int* list = p.idx + row * p.keep;
    const long long base = (row / g.H) * g.sb + (row % g.H) * g.sh + sub * 8;
    const long long orow = row * p.keep;
    int tn[U];
#pragma unroll
    for (int u = 0; u < U; ++u) tn[u] = __ldcg(list + min(j0 + u * GPB + grp, j1 - 1));
    for (int jb = j0; jb < j1; jb += GPB * U) {
        int t[U];
#pragma unroll
        for (int u = 0; u < U; ++u) t[u] = tn[u];
        if (jb + GPB * U < j1) {   // block-uniform
#pragma unroll
            for (int u = 0; u < U; ++u) tn[u] = __ldcg(list + min(jb + GPB * U + u * GPB + grp, j1 - 1));
        }
        uint4 kr[U], vr[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {   // rows past the end repeat the slice's last row; only their stores are dropped
            const long long src = base + (long long)SKV_INDEX(max(t[u], 0), p.T) * g.st;
            kr[u] = ld_stream16(g.k + src);
            vr[u] = ld_stream16(g.v + src);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int j = jb + u * GPB + grp;
            const bool valid = j < j1;
            const long long r = orow + j;
            if (MODE == SKV_QUANT_NONE) {
                quant_row<MODE>(kr[u], sub, LPR, nullptr, nullptr, static_cast<__half*>(g.k_out) + r * D, valid);
                quant_row<MODE>(vr[u], sub, LPR, nullptr, nullptr, static_cast<__half*>(g.v_out) + r * D, valid);
            } else {
                quant_row<MODE>(kr[u], sub, LPR, static_cast<uint8_t*>(g.k_out) + r * D, g.k_scale + r, nullptr, valid);
                quant_row<MODE>(vr[u], sub, LPR, static_cast<uint8_t*>(g.v_out) + r * D, g.v_scale + r, nullptr, valid);
            }
        }
    }
    SKV_PHASE(11);
}

template <int D>
static int launch_fused(const SelectParams& sp, const GatherParams& gp, int mode, long long rows, cudaStream_t st) {
    const dim3 grid((unsigned)(rows * CL)), block(SEL_THREADS);
    switch (mode) {
        case SKV_QUANT_NONE: evict_fused_cluster_kernel<D, SKV_QUANT_NONE><<<grid, block, 0, st>>>(sp, gp); break;
        case SKV_QUANT_INT8: evict_fused_cluster_kernel<D, SKV_QUANT_INT8><<<grid, block, 0, st>>>(sp, gp); break;
        case SKV_QUANT_E4M3: evict_fused_cluster_kernel<D, SKV_QUANT_E4M3><<<grid, block, 0, st>>>(sp, gp); break;
        default: evict_fused_cluster_kernel<D, SKV_QUANT_CAST><<<grid, block, 0, st>>>(sp, gp); break;
    }
    SKV_CUDA_TRY(cudaGetLastError());
    return SKV_OK;
}

inline int& fused_flag() { static int on = 0; return on; }   // two launches measure faster on B200 (see skv_kv_evict_set_fused)
inline bool fused_enabled() { return fused_flag() != 0; }

static size_t select_smem() { return (size_t)TopkSmem<SEL_THREADS>::WORDS * 4 + (size_t)MAX_KEEP * 8; }

template <int D>
static int launch_gather(const GatherParams& gp, int mode, int device, cudaStream_t st) {
    constexpr int GPB = GQ_THREADS / (D / 8);
    const long long rows = gp.rows_total / gp.keep;               // B * H
    if (rows > 65535) return fail(SKV_ERR_UNSUPPORTED, "B * H = %lld exceeds 65535", rows);
    int chunks = (gp.keep + GPB * 4 - 1) / (GPB * 4);             // U = 4 rows per group and step
#ifndef SKV_GATHER_CAP
#define SKV_GATHER_CAP 16
#endif
    const long long cap = ((long long)sm_count(device) * SKV_GATHER_CAP + rows - 1) / rows;   // CTAs per (b, h)
    if (chunks > cap) chunks = (int)(cap > 0 ? cap : 1);
    const dim3 grid((unsigned)chunks, (unsigned)rows), block(GQ_THREADS);
    switch (mode) {
        case SKV_QUANT_NONE: SKV_CUDA_TRY(launch_pdl(evict_gather_quant_kernel<D, SKV_QUANT_NONE>, grid, block, 0, st, gp)); break;
        case SKV_QUANT_INT8: SKV_CUDA_TRY(launch_pdl(evict_gather_quant_kernel<D, SKV_QUANT_INT8>, grid, block, 0, st, gp)); break;
        case SKV_QUANT_E4M3: SKV_CUDA_TRY(launch_pdl(evict_gather_quant_kernel<D, SKV_QUANT_E4M3>, grid, block, 0, st, gp)); break;
        default: SKV_CUDA_TRY(launch_pdl(evict_gather_quant_kernel<D, SKV_QUANT_CAST>, grid, block, 0, st, gp)); break;
    }
    SKV_CUDA_TRY(cudaGetLastError());
    return SKV_OK;
}

}  // namespace evq
}  // namespace skv

using namespace skv;

extern "C" {

// Number of rows kept per head: min(budget, T - recent') + recent' with recent' = min(recent, T).
int skv_kv_evict_keep_count(int T, int budget, int recent) {
    if (T <= 0 || budget < 0 || recent < 0) return 0;
    const int r = recent < T ? recent : T;
    const int kb = budget < T - r ? budget : T - r;
    return kb + r;
}

#ifdef SKV_PROFILE_PHASES
int skv_debug_phase_ts_evict(unsigned long long* out) {
    return cudaMemcpyFromSymbol(out, skv_phase_ts, sizeof(unsigned long long) * 32) == cudaSuccess ? 0 : -4;
}
#endif

// 1: the single-launch cluster kernel serves the cases it covers; 0 (default): select and gather in two launches.
int skv_kv_evict_set_fused(int on) {
    evq::fused_flag() = on ? 1 : 0;
    return SKV_OK;
}

int skv_kv_evict_quant(const void* k_cache, const void* v_cache, const float* scores, int* idx_out,
                       void* k_out, void* v_out, float* k_scale_out, float* v_scale_out,
                       int B, int H, int T, int D, long long kv_stride_b, long long kv_stride_h,
                       long long kv_stride_t, int budget, int recent, int quant_mode, int order, int device,
                       void* stream) {
    if (!k_cache || !v_cache || !scores || !idx_out || !k_out || !v_out)
        return fail(SKV_ERR_BAD_ARG, "skv_kv_evict_quant: null tensor pointer");
    if (B <= 0 || H <= 0 || T <= 0) return fail(SKV_ERR_BAD_ARG, "skv_kv_evict_quant: sizes must be positive");
    if (budget < 0 || recent < 0) return fail(SKV_ERR_BAD_ARG, "budget and recent must not be negative");
    if (D != 16 && D != 32 && D != 64 && D != 128 && D != 256)
        return fail(SKV_ERR_UNSUPPORTED, "head dim %d not supported (16, 32, 64, 128 or 256)", D);
    if (quant_mode < SKV_QUANT_NONE || quant_mode > SKV_QUANT_CAST) return fail(SKV_ERR_BAD_ARG, "unknown quant_mode %d", quant_mode);
    if (order != SKV_ORDER_POSITION && order != SKV_ORDER_SCORE) return fail(SKV_ERR_BAD_ARG, "unknown order %d", order);
    if ((quant_mode == SKV_QUANT_INT8 || quant_mode == SKV_QUANT_E4M3) && (!k_scale_out || !v_scale_out))
        return fail(SKV_ERR_BAD_ARG, "scaled quantisation needs k_scale_out and v_scale_out");
    const int keep = skv_kv_evict_keep_count(T, budget, recent);
    if (keep <= 0) return fail(SKV_ERR_BAD_ARG, "nothing to keep (budget + recent == 0)");
    if (keep > evq::MAX_KEEP) return fail(SKV_ERR_UNSUPPORTED, "keep count %d exceeds %d", keep, evq::MAX_KEEP);
    if ((kv_stride_t % 8) || (kv_stride_h % 8) || (kv_stride_b % 8))
        return fail(SKV_ERR_BAD_ARG, "strides must be multiples of 8 elements (16-byte rows)");
    if ((reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) | reinterpret_cast<uintptr_t>(k_out) |
         reinterpret_cast<uintptr_t>(v_out)) & 15)
        return fail(SKV_ERR_BAD_ARG, "cache and output pointers must be 16-byte aligned");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(SKV_ERR_CUDA, "cannot switch to device %d", device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    static bool configured[64] = {false};
    const size_t smem = evq::select_smem();
    if (device < 64 && !configured[device]) {
        SKV_CUDA_TRY(cudaFuncSetAttribute(evq::evict_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured[device] = true;
    }
    evq::SelectParams sp;
    sp.scores = scores; sp.idx = idx_out; sp.T = T; sp.budget = budget; sp.recent = recent; sp.keep = keep; sp.order = order;
    evq::GatherParams gp;
    gp.k = static_cast<const __half*>(k_cache);
    gp.v = static_cast<const __half*>(v_cache);
    gp.idx = idx_out;
    gp.k_out = k_out; gp.v_out = v_out; gp.k_scale = k_scale_out; gp.v_scale = v_scale_out;
    gp.H = H; gp.keep = keep; gp.T = T; gp.rows_total = (long long)B * H * keep;
    gp.sb = kv_stride_b; gp.sh = kv_stride_h; gp.st = kv_stride_t;

    const int competing = T - (recent < T ? recent : T);
    const bool cluster_ok = order == SKV_ORDER_POSITION && competing <= evq::CL * evq::SEL_THREADS * evq::KR &&
                            (long long)B * H * evq::CL <= 65535LL * 32;
    if (cluster_ok && evq::fused_enabled() && (D == 128 || D == 64)) {   // one launch: select, then gather by the same cluster
        return D == 128 ? evq::launch_fused<128>(sp, gp, quant_mode, (long long)B * H, st)
                        : evq::launch_fused<64>(sp, gp, quant_mode, (long long)B * H, st);
    }
    if (cluster_ok) {
        evq::evict_select_cluster_kernel<<<(unsigned)((long long)B * H * evq::CL), evq::SEL_THREADS, 0, st>>>(sp);
    } else {
        evq::evict_select_kernel<<<(unsigned)((long long)B * H), evq::SEL_THREADS, smem, st>>>(sp);
    }
    SKV_CUDA_TRY(cudaGetLastError());
    switch (D) {
        case 16: return evq::launch_gather<16>(gp, quant_mode, device, st);
        case 32: return evq::launch_gather<32>(gp, quant_mode, device, st);
        case 64: return evq::launch_gather<64>(gp, quant_mode, device, st);
        case 128: return evq::launch_gather<128>(gp, quant_mode, device, st);
        default: return evq::launch_gather<256>(gp, quant_mode, device, st);
    }
}

}  // extern "C"

SKV_BOUNDS_GETTER(skv_debug_bounds_kv_evict)
