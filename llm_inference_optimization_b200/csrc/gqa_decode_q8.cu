// Dense GQA decode attention over a PAGED 8-bit KV cache (INT8 or FP8-E4M3 codes
// with one fp32 scale per token and kv-head), dequantisation fused into the kernel.
//
// No reference counterpart: the reference kernel reads an unpaged fp16 cache only
// (csrc/kernels/gqa_decode.cu:84-90) and its INT8 path is disabled
// (csrc/kernels/kv_evict_quant.cu:294).  The arithmetic is
//   Out[b,hq] = softmax_t(scale * ks[t] * q . kc[t]) . (vs[t] * vc[t])
// with kc/vc the stored codes and ks/vs their scales.
//
// Cache layout: code pools addressed (page, kv-head, slot, channel) with D = 128
// one-byte channels per row; scale pools (page, kv-head, slot) fp32;
// page_table[b, i] gives the physical page of tokens [i*P, (i+1)*P) of sequence b.
// P (tokens per page) is a multiple of 16; an unpaged [B, H, T, D] cache is the
// special case P = T with a null page table.
//
// Same skeleton as the fp16 kernel: grid (Hkv, splits, B), producers feeding a ring
// of 64-token stages through mbarriers, consumers with mma.sync, online softmax,
// in-CTA merge, ticketed split combine.  Differences:
//   * four producer warps share every stage (an async copy costs its issuing warp
//     100-200 cycles); a stage is four fused page records (one TMA box each), or K/V
//     boxes plus bulk copies of the scales for separate pools; page ids are
//     prefetched 32 tiles ahead, one per lane;
//   * NG groups of four consumer warps work on the stages in turn: two groups in one 384-thread CTA per SM, or
//     one group in 256-thread CTAs of which two share an SM (so that one streams while the other starts or ends);
//   * tokens are on the M side of both products (S^T = K Q^T, O^T = V^T P^T) and the
//     query heads on the 8-wide N side: a group of <= 8 heads needs one n-tile;
//     P is moved to the B-operand layout with movmatrix;
//   * codes are converted to fp16 in registers right after ldmatrix (e4m3x2 ->
//     f16x2 by cvt; int8 by a byte-permute into the mantissa of 1024 + x, whose bias is taken out of the
//     accumulators instead of every element, see cvt_quad_k); because four bytes arrive
//     per lane where an fp16 fragment has two halves, the contraction index of
//     S^T and the output channels of O^T are permuted consistently;
//   * ks[t] multiplies the fp32 score; vs[t] (times 2^6, undone at the end, to stay
//     clear of fp16 subnormals) is folded into P before it is rounded to fp16.
#include <cuda_fp8.h>

#include "gqa_epilogue.cuh"
#include "skv_common.cuh"
#include "skv_tmap.cuh"

namespace skv {
namespace gqa {

constexpr int Q8_D = 128;
constexpr int CHUNK = 16;                                  // tokens per TMA box / scale copy
constexpr int Q8_CODE_BYTES = TILE * Q8_D;                 // 8 KB of K (or V) codes per stage
constexpr int Q8_STAGE_BYTES = 2 * Q8_CODE_BYTES + 1024;   // + K scales [64] + V scales [64] (512 B, padded)
constexpr float P_BOOST = 64.f;
// How a 64-token stage is fetched.  Every async copy costs its issuing lane about 100 cycles, so a stage
// should be made of few requests:
//   Q8_SEPARATE16: four 16-token chunks, each a K box, a V box and two 64-byte scale copies (16 requests);
//   Q8_SEPARATE64: pages of a multiple of 64 tokens: one K box, one V box, two 256-byte scale copies;
//   Q8_FUSED     : "page records" -- K codes, V codes and both scale vectors of a (page, head) stored as
//                  33 consecutive 128-byte rows, fetched by ONE box per 16-token chunk (4 requests).
constexpr int Q8_SEPARATE16 = 0, Q8_SEPARATE64 = 1, Q8_FUSED = 2;
constexpr int RECORD_ROWS = 33;                            // 16 K rows, 16 V rows, 1 row of 16 + 16 fp32 scales
constexpr int RECORD_BYTES = RECORD_ROWS * Q8_D;           // 4224
// Mixed-precision page records: K in 8 bits, V in 4 (two channels per byte, 64 bytes per token, two tokens per
// 128-byte row): 16 K rows, 8 V rows, 1 row of scales.  A stage of four such records is padded to a multiple of
// 1 KB so that every stage starts at the same phase of the 128-byte swizzle.
constexpr int V4_RECORD_ROWS = 25;
constexpr int V4_RECORD_BYTES = V4_RECORD_ROWS * Q8_D;     // 3200
constexpr int V4_STAGE_BYTES = 13 * 1024;                  // 4 * 3200 = 12800, padded
// A 4-bit V code is stored as u = q + 8 (q in -7..7); 0x6400 | u is the fp16 number q + 1032, and the 1032 is taken
// out of the accumulators like the INT8 bias (see cvt_quad_k).
constexpr float V4_BIAS = 1032.f;
// Consumer groups of four warps; group g takes the stages with it % groups == g.  The ring depth must be a
// multiple of the group count so that a stage always belongs to the same group: a group that could reach a
// stage two uses ahead of another group's wait would pass a parity wait meant for the use before.  Two groups
// are enough (a third, tried with 123 registers per thread, brought no gain at 16 x 64K).
// A one-group variant (256 threads, <= 128 registers, 6 stages) fits two CTAs on an SM, so that one streams while
// the other is in its prologue or epilogue.  It is used for FP8 caches when a launch has many CTAs per SM
// (16 x 64K: 379 -> 350 us); the INT8 conversion costs the consumers more and keeps two groups per CTA.
constexpr int Q8_PRODUCERS = 4;                            // producer warps: each issues one share of every stage
__host__ __device__ constexpr int q8_threads(int ng) { return (ng * CONSUMER_WARPS + Q8_PRODUCERS) * 32; }

#ifdef SKV_PROFILE_PHASES
static __device__ unsigned long long skv_cta_ts[5][1024];
#define SKV_CTA_STAMP(slot)                                                                              \
    do {                                                                                                 \
        const unsigned lin_ = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);            \
        if ((threadIdx.x & 31) == 0 && lin_ < 1024) {                                                    \
            unsigned long long t_;                                                                       \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                       \
            if ((slot) == 0 || (slot) == 1) atomicMin(&skv_cta_ts[slot][lin_], t_);                      \
            else atomicMax(&skv_cta_ts[slot][lin_], t_);                                                 \
            if ((slot) == 0) { unsigned sm_; asm volatile("mov.u32 %0, %%smid;" : "=r"(sm_)); skv_cta_ts[4][lin_] = sm_; } \
        }                                                                                                \
    } while (0)
#else
#define SKV_CTA_STAMP(slot) do {} while (0)
#endif

struct Q8Params {
    const __half* q;
    __half* out;
    float* partial_o;
    float* partial_ml;
    int* tickets;
    int* status;
    const int* seq_lens;     // [B] or null
    const int* page_table;   // [B, max_pages] or null (then page = b * max_pages + i)
    const float* k_scale;    // element (page, h, slot) at page*sc_sp + h*sc_sh + slot
    const float* v_scale;
    int N, Hq, Hkv, G;
    int tiles_per_split, num_splits, stages;
    int page_size, max_pages;
    int num_pages;           // pages in the pools: ids read from the table are checked against it
    int list_items;          // > 0: grid.y indexes a work list of (sequence, split) items built from seq_lens (see the kernel); 0: grid (Hkv, splits, B)
    int B;                   // sequences (the work-list mode has no batch dimension in its grid)
    int mode;                // Q8_SEPARATE16, Q8_SEPARATE64 or Q8_FUSED
    int out_bf16;            // output elements are bf16 instead of fp16
    int early_kv;            // 1: pages, page table and seq_lens are not produced by the previous kernel; 2: the same except
                             // for each sequence's LAST token (appended by the previous kernel): its tile waits
    long long sc_sp, sc_sh;
    long long q_stride_b, q_stride_h, o_stride_b, o_stride_h;
    float scale_log2;
    PoolMapPos pos;
};

template <int NG, bool V4 = false>
static size_t q8_smem_bytes(int stages) {
    size_t ring = (size_t)stages * (V4 ? V4_STAGE_BYTES : Q8_STAGE_BYTES);
    size_t merge = merge_smem_bytes<Q8_D, NG * CONSUMER_WARPS>();
    return 1024 + (ring > merge ? ring : merge) + 2 * stages * 8 + 16;
}

// Four 8-bit codes [c0,c1,c2,c3] in one register -> half2(c0,c1) and half2(c2,c3).
template <int KVT>
__device__ __forceinline__ void cvt_quad(uint32_t v, uint32_t& lo, uint32_t& hi) {
    if (KVT == SKV_KV_E4M3) {
        asm("{\n\t.reg .b16 a, b;\n\tmov.b32 {a, b}, %2;\n\t"
            "cvt.rn.f16x2.e4m3x2 %0, a;\n\tcvt.rn.f16x2.e4m3x2 %1, b;\n\t}"
            : "=r"(lo), "=r"(hi)
            : "r"(v));
    } else {
        // int8 b -> fp16: 0x6400 | (b ^ 0x80) is exactly 1024 + (b + 128); subtract 1152
        const uint32_t x = v ^ 0x80808080u;
        uint32_t a = __byte_perm(x, 0x64646464u, 0x4140), b = __byte_perm(x, 0x64646464u, 0x4342);
        const __half2 bias = __float2half2_rn(1152.f);
        const __half2 ra = __hsub2(*reinterpret_cast<__half2*>(&a), bias);
        const __half2 rb = __hsub2(*reinterpret_cast<__half2*>(&b), bias);
        lo = *reinterpret_cast<const uint32_t*>(&ra);
        hi = *reinterpret_cast<const uint32_t*>(&rb);
    }
}

// The same for the tensor-core operands, where INT8 codes keep the bias of the exponent trick: 0x6400 | (b ^ 0x80) is
// the fp16 number b + 1152, and instead of subtracting 1152 from every element (two HSUB2 per four codes, more than the
// conversion itself) the products are corrected once per accumulator:
//     sum_d q_d (k_d + 1152) = q.k + 1152 sum_d q_d          (per head: a constant of the launch)
//     sum_t p_t (v_t + 1152) = p.v + 1152 sum_t p_t          (per head: one more MMA per step, against a tile of ones)
// Every product is exact in fp32 (11-bit q or p times an integer below 2048).  cvt_quad_v also folds in the byte
// shuffle of the transposed V tile ([c0, c2 | c1, c3] of the register).
constexpr float INT8_BIAS = 1152.f;

// (a & b) | c in one LOP3
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

template <int KVT>
__device__ __forceinline__ void cvt_quad_k(uint32_t v, uint32_t& lo, uint32_t& hi) {
    if (KVT == SKV_KV_E4M3) {
        cvt_quad<KVT>(v, lo, hi);
    } else {
        const uint32_t x = v ^ 0x80808080u;
        lo = __byte_perm(x, 0x64646464u, 0x4140);
        hi = __byte_perm(x, 0x64646464u, 0x4342);
    }
}

template <int KVT>
__device__ __forceinline__ void cvt_quad_v(uint32_t v, uint32_t& lo, uint32_t& hi) {
    if (KVT == SKV_KV_E4M3) {
        cvt_quad<KVT>(__byte_perm(v, 0u, 0x3120), lo, hi);
    } else {
        const uint32_t x = v ^ 0x80808080u;
        lo = __byte_perm(x, 0x64646464u, 0x4240);
        hi = __byte_perm(x, 0x64646464u, 0x4341);
    }
}

__device__ __forceinline__ void pool_tile_load(uint32_t dst, const CUtensorMap* tm, uint32_t bar, const PoolMapPos& pos,
                                               int slot, int head, int page, uint64_t policy) {
    int c[4] = {0, 0, 0, 0};
#pragma unroll
    for (int i = 1; i < 4; ++i) c[i] = (i == pos.slot) ? slot : (i == pos.head) ? head : page;
    tma_load_4d(dst, tm, bar, c[0], c[1], c[2], c[3], policy);
}

template <int KVT, int NT, int NG, bool V4 = false>
__global__ void __launch_bounds__(q8_threads(NG), NG == 1 ? 2 : 1)
gqa_decode_q8_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                     const Q8Params p) {
    constexpr int D = Q8_D;
    constexpr int STAGE_BYTES = V4 ? V4_STAGE_BYTES : Q8_STAGE_BYTES;     // V4: fused records only
    constexpr int REC_BYTES = V4 ? V4_RECORD_BYTES : RECORD_BYTES;
    constexpr bool V_BIASED = V4 || KVT != SKV_KV_E4M3;                   // V operand carries an additive bias
    constexpr float V_BIAS = V4 ? V4_BIAS : INT8_BIAS;
    constexpr int Q8_GROUPS = NG;
    constexpr int Q8_WARPS = Q8_GROUPS * CONSUMER_WARPS;
    constexpr int Q8_CONSUMER_THREADS = Q8_WARPS * 32;
    constexpr int NCH = D / 16;  // 16-byte chunks per row = MMA k-steps of S = Q K^T
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.x;
    int split = blockIdx.y, b = blockIdx.z;
    SKV_PHASE(0);
    SKV_CTA_STAMP(0);

    // Ordered like any other kernel unless the caller declared the cache static (see the fp16 kernel).
    if (!p.early_kv) pdl_wait_prior_grids();
    SKV_PHASE(1);
    int len, tiles_per_split = p.tiles_per_split, n_splits;
    if (p.list_items > 0) {   // work-list schedule of a ragged batch (see worklist_item)
        const SplitItem it = worklist_item(p.seq_lens, p.B, p.N, p.list_items, blockIdx.y, p.tiles_per_split);
        if (it.b < 0) return;
        b = it.b; split = it.split; len = it.len; n_splits = it.n_splits; tiles_per_split = it.tiles_per_split;
    } else {
        len = p.seq_lens ? min(max(p.seq_lens[b], 0), p.N) : p.N;
        const int tps_tokens = tiles_per_split * TILE;
        n_splits = len > 0 ? (len + tps_tokens - 1) / tps_tokens : 1;
        if (split >= n_splits) return;
    }
    const int tokens_per_split = tiles_per_split * TILE;
    const int t_begin = split * tokens_per_split;
    const int t_end = min(len, t_begin + tokens_per_split);
    const int ntiles = (t_end - t_begin + TILE - 1) / TILE;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t ring = smem_u32(smem);
    size_t body = (size_t)p.stages * STAGE_BYTES;
    if (merge_smem_bytes<D, Q8_WARPS>() > body) body = merge_smem_bytes<D, Q8_WARPS>();
    const uint32_t full_bar = ring + (uint32_t)body;
    const uint32_t empty_bar = full_bar + p.stages * 8;
    int* last_flag = reinterpret_cast<int*>(smem + body + 2 * p.stages * 8);

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(full_bar + s * 8, Q8_PRODUCERS);
            mbar_init(empty_bar + s * 8, CONSUMER_WARPS);
        }
        fence_barrier_init();
    }
    __syncthreads();

    // ------------------------------------------------------------------ producers
    // Issuing one async copy costs its warp 100-200 cycles, and the copies of one warp are issued one after
    // another, so a single producer warp cannot keep up with the ~700 cycles a 64-token stage lasts at full
    // HBM rate.  Four producer warps therefore share every stage; each waits for the stage to be free, adds
    // its own byte count to the stage's full-barrier (arrival count Q8_PRODUCERS) and issues its copies:
    //   16-token request groups (fused records / separate pools): warp w fetches chunk w of the stage;
    //   64-token boxes: warp 0 the K box, 1 the V box, 2 the K scales, 3 the V scales.
    // Lane l of a producer warp resolves the page of tile (batch * 32 + l) ahead of time, one page-table
    // read per lane per 32 tiles; lane 0 does the waiting and issuing.
    if (warp >= Q8_WARPS) {
        const int pw = warp - Q8_WARPS;
        if (lane == 0 && pw == 0) {
            tma_prefetch_desc(&tmK);
            tma_prefetch_desc(&tmV);
        }
        const uint64_t policy = l2_policy_evict_first();
        const int P = p.page_size;
        const bool big = p.mode == Q8_SEPARATE64;
        const int tok_off = big ? 0 : pw * CHUNK;                 // first token of this warp's share inside a stage
        const uint32_t my_tx = p.mode == Q8_FUSED ? (uint32_t)REC_BYTES
                             : big ? (pw < 2 ? (uint32_t)(TILE * D) : (uint32_t)(TILE * 4))
                                   : (uint32_t)(2 * CHUNK * D + 2 * CHUNK * 4);
        int s = 0;
        uint32_t ph = 0;
        int ok = 1;
        bool bad_page = false;
        bool waited_for_append = false;
        for (int it0 = 0; it0 < ntiles && ok; it0 += 32) {
            int page = -1, slot = 0;
            {
                const int t = t_begin + (it0 + lane) * TILE + tok_off;
                if (t < t_end) {
                    const int lp = t / P;
                    slot = t - lp * P;
                    page = p.page_table ? __ldg(p.page_table + (long long)b * p.max_pages + lp) : b * p.max_pages + lp;
                    // A page id outside the pools (a stale or corrupt table entry) must not become an address:
                    // page 0 is read in its place, so the output stays finite, and the status word says so.
                    page = checked_page(page, p.num_pages, bad_page);
                }
            }
            const int jn = min(32, ntiles - it0);
            for (int j = 0; j < jn; ++j) {
                const int pg = __shfl_sync(0xffffffffu, page, j), sl = __shfl_sync(0xffffffffu, slot, j);
                // early_kv == 2: the previous kernel in the stream stores the sequence's last token (position len - 1);
                // every tile before the one that holds it streams at once, that one only after the kernel is done
                if (p.early_kv == 2 && !waited_for_append && t_begin + (it0 + j + 1) * TILE >= len) {
                    pdl_wait_prior_grids();
                    waited_for_append = true;
                }
                if (lane == 0) {
                    const uint32_t bar = full_bar + s * 8;
                    if (it0 + j >= p.stages && !mbar_wait(empty_bar + s * 8, ph ^ 1u)) {
                        atomicOr(p.status, SKV_DEV_TIMEOUT);
                        ok = 0;
                    } else if (pg < 0) {
                        mbar_arrive(bar);                         // nothing of this warp's share lies inside the sequence
                    } else {
                        mbar_expect_tx(bar, my_tx);
                        const uint32_t kdst = ring + s * STAGE_BYTES;
                        const long long so = (long long)pg * p.sc_sp + (long long)h * p.sc_sh + sl;
                        if (p.mode == Q8_FUSED) {
                            pool_tile_load(kdst + pw * REC_BYTES, &tmK, bar, p.pos, 0, h, pg, policy);
                        } else if (big) {
                            if (pw == 0) pool_tile_load(kdst, &tmK, bar, p.pos, sl, h, pg, policy);
                            else if (pw == 1) pool_tile_load(kdst + Q8_CODE_BYTES, &tmV, bar, p.pos, sl, h, pg, policy);
                            else bulk_load(kdst + 2 * Q8_CODE_BYTES + (pw == 3 ? 256 : 0), (pw == 2 ? p.k_scale : p.v_scale) + so, TILE * 4, bar);
                        } else {
                            pool_tile_load(kdst + tok_off * D, &tmK, bar, p.pos, sl, h, pg, policy);
                            pool_tile_load(kdst + Q8_CODE_BYTES + tok_off * D, &tmV, bar, p.pos, sl, h, pg, policy);
                            bulk_load(kdst + 2 * Q8_CODE_BYTES + tok_off * 4, p.k_scale + so, CHUNK * 4, bar);
                            bulk_load(kdst + 2 * Q8_CODE_BYTES + 256 + tok_off * 4, p.v_scale + so, CHUNK * 4, bar);
                        }
                    }
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                if (++s == p.stages) { s = 0; ph ^= 1u; }
            }
        }
        report_bad_page(bad_page, p.status);
        return;
    }

    // ----------------------------------------------------------------- consumers
    // The query, the workspace and the output may belong to the previous kernel until now (early_kv mode; otherwise
    // the whole CTA has already waited).  The next launch is released only after this wait: it then starts after
    // everything older than this kernel has completed, and this kernel writes no K/V.
    if (p.early_kv) pdl_wait_prior_grids();
    pdl_launch_dependents();
    // Tokens sit on the M side of both products (S^T = K Q^T, O^T = V^T P^T) and the query heads on the 8-wide N
    // side, so a group of up to 8 heads costs one n-tile (NT = 1) instead of a mostly empty 16-row M tile.
    const int g = lane >> 2, tq = lane & 3;
    const int G = p.G;

    // Query as the B operand.  Lane (g, tq) receives bytes 4tq..4tq+3 of every 16-byte chunk c of a key row, so
    // MMA k-index 2tq+{0,1} of k-step c stands for channel 16c+4tq+{0,1} and k-index 2tq+8+{0,1} for 16c+4tq+{2,3};
    // column n of n-tile nt is head 8nt + n.
    uint32_t qb[NT][NCH][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const int head = nt * 8 + g;
        const __half* qrow = p.q + (long long)b * p.q_stride_b + (long long)(h * G + head) * p.q_stride_h + tq * 4;
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
            const uint2 v = head < G ? *reinterpret_cast<const uint2*>(qrow + c * 16) : make_uint2(0u, 0u);
            qb[nt][c][0] = v.x;
            qb[nt][c][1] = v.y;
        }
    }

    // INT8: 1152 * (sum of the query's channels) for this lane's two score columns, heads 8nt+2tq and 8nt+2tq+1
    float qbias[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        qbias[nt][0] = qbias[nt][1] = 0.f;
        if (KVT != SKV_KV_E4M3) {
            float sum = 0.f;
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                const float2 u = __half22float2(*reinterpret_cast<const __half2*>(&qb[nt][c][0]));
                const float2 w = __half22float2(*reinterpret_cast<const __half2*>(&qb[nt][c][1]));
                sum += (u.x + u.y) + (w.x + w.y);
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);          // lanes (g, *): all channels of head 8nt+g
            qbias[nt][0] = INT8_BIAS * __shfl_sync(0xffffffffu, sum, (2 * tq) * 4);
            qbias[nt][1] = INT8_BIAS * __shfl_sync(0xffffffffu, sum, (2 * tq + 1) * 4);
        }
    }

    // o[nt][c][j], o[nt][c][j+2]: channels 16c+2g and 16c+2g+1 of head 8nt+2tq+j
    float o[NT][NCH][4];
    float psum[NT][4];   // INT8: sum over tokens of the P operand, in o's layout (every channel row the same)
    float mrun[NT][2], lrun[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int c = 0; c < NCH; ++c) o[nt][c][0] = o[nt][c][1] = o[nt][c][2] = o[nt][c][3] = 0.f;
        mrun[nt][0] = mrun[nt][1] = -INFINITY;
        lrun[nt][0] = lrun[nt][1] = 0.f;
        psum[nt][0] = psum[nt][1] = psum[nt][2] = psum[nt][3] = 0.f;
    }
    const int lj = lane >> 3, r8 = lane & 7;
    const int group = warp >> 2;          // consumer group: takes the stages with it % Q8_GROUPS == group
    const int wc = warp & 3;              // this warp's 16-token chunk of a stage
    const int wtok = wc * 16;
    // Byte offsets inside a stage of this warp's 16 K rows, 16 V rows and 16 + 16 scales, and the swizzle
    // phase of its first row (rows are 128 bytes; TMA XORs the 16-byte chunk index with the row index mod 8).
    const bool fused = p.mode == Q8_FUSED;
    const uint32_t k_off = fused ? wc * REC_BYTES : wtok * D;
    const uint32_t v_off = fused ? wc * REC_BYTES + 16 * D : Q8_CODE_BYTES + wtok * D;
    const uint32_t ks_off = fused ? wc * REC_BYTES + (V4 ? 24 : 32) * D : 2 * Q8_CODE_BYTES + wtok * 4;
    const uint32_t vs_off = fused ? ks_off + 64 : ks_off + 256;
    const int sc_phase = fused ? wc : 0;                  // the scale row of a record is swizzled too
    const uint32_t sw = (uint32_t)((r8 + (fused ? wc : 0)) & 7);
    // ldmatrix x4 addressing, the same for K and V: matrices (tokens 0-7, chunk c), (tokens 8-15, chunk c),
    // (tokens 0-7, chunk c+1), (tokens 8-15, chunk c+1)
    const uint32_t ld_row_off = (uint32_t)(((lj & 1) * 8 + r8) * 128);
    const uint32_t ld_ch = (uint32_t)(lj >> 1);
    // 4-bit V rows hold two tokens (64 bytes each): the lane's token (lj & 1) * 8 + r8 sits in row token / 2 at chunk
    // (token & 1) * 4 + (32-channel chunk), swizzled with that row's phase
    const int v4_tok = (lj & 1) * 8 + r8;
    const uint32_t v4_row_off = (uint32_t)((v4_tok >> 1) * 128);
    const uint32_t v4ch = (uint32_t)((v4_tok & 1) * 4 + (lj >> 1));
    const uint32_t v4sw = (uint32_t)(((v4_tok >> 1) + wc) & 7);
    // scales of this lane's two tokens (rows g and g+8 of the warp's 16)
    const uint32_t sc_off0 = (uint32_t)(((((g) >> 2) ^ sc_phase) << 4) + (g & 3) * 4);
    const uint32_t sc_off1 = (uint32_t)(((((g + 8) >> 2) ^ sc_phase) << 4) + (g & 3) * 4);

    int s = group;          // stage of tile `it`; p.stages >= Q8_GROUPS, so one wrap per step at most
    uint32_t ph = 0;
    SKV_PHASE(2);
    for (int it = group; it < ntiles; it += Q8_GROUPS, s += Q8_GROUPS) {
        if (s >= p.stages) { s -= p.stages; ph ^= 1u; }
        if (!mbar_wait(full_bar + s * 8, ph)) {
            if (lane == 0) atomicOr(p.status, SKV_DEV_TIMEOUT);
            break;
        }
        if (it == group) { SKV_PHASE(3); SKV_CTA_STAMP(1); }
        const int tok0 = t_begin + it * TILE + wtok;
        if (tok0 < t_end) {
            const uint32_t kbase = ring + s * STAGE_BYTES + k_off + ld_row_off;   // this lane's K row
            const uint32_t vbase = ring + s * STAGE_BYTES + v_off + ld_row_off;   // this lane's V row
            const uint32_t v4base = ring + s * STAGE_BYTES + v_off + v4_row_off;  // this lane's row of 4-bit V codes
            const uint8_t* stage = smem + (size_t)s * STAGE_BYTES;
            const bool ragged = tok0 + 16 > t_end;
            if (ragged && !V4) {   // (4-bit codes are integers: a stale row times a zero weight is zero)
                // rows past the end hold stale bytes (possibly NaN codes): zero them in V
                for (int idx = lane; idx < 16 * 8; idx += 32) {
                    const int r = idx >> 3, c = idx & 7;
                    if (tok0 + r >= t_end)
                        *reinterpret_cast<uint4*>(smem + (size_t)s * STAGE_BYTES + v_off + (size_t)r * 128 +
                                                  (size_t)c * 16) = make_uint4(0u, 0u, 0u, 0u);
                }
                __syncwarp();
            }

            // S^T = K Q^T: two accumulators per n-tile (even / odd k-steps) halve the dependent MMA chain
            float sc[NT][4], sd[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) sc[nt][j] = sd[nt][j] = 0.f;
#pragma unroll
            for (int m = 0; m < NCH / 2; ++m) {
                uint32_t r0, r1, r2, r3;
                ldsm_x4(kbase + (((uint32_t)(2 * m) + ld_ch) ^ sw) * 16, r0, r1, r2, r3);
                uint32_t a0[4], a1[4];
                cvt_quad_k<KVT>(r0, a0[0], a0[2]);   // token g:   k-indices 2tq.. and 2tq+8..
                cvt_quad_k<KVT>(r1, a0[1], a0[3]);   // token g+8
                cvt_quad_k<KVT>(r2, a1[0], a1[2]);
                cvt_quad_k<KVT>(r3, a1[1], a1[3]);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    mma_f16(sc[nt], a0, qb[nt][2 * m][0], qb[nt][2 * m][1]);
                    mma_f16(sd[nt], a1, qb[nt][2 * m + 1][0], qb[nt][2 * m + 1][1]);
                }
            }
            float ks0 = *reinterpret_cast<const float*>(stage + ks_off + sc_off0) * p.scale_log2;
            float ks1 = *reinterpret_cast<const float*>(stage + ks_off + sc_off1) * p.scale_log2;
            float vs0 = *reinterpret_cast<const float*>(stage + vs_off + sc_off0) * P_BOOST;
            float vs1 = *reinterpret_cast<const float*>(stage + vs_off + sc_off1) * P_BOOST;
            const bool dead0 = ragged && tok0 + g >= t_end, dead1 = ragged && tok0 + g + 8 >= t_end;
            if (dead0) vs0 = 0.f;
            if (dead1) vs1 = 0.f;
            float mnew[NT][2];
            bool grow = false;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                if (KVT != SKV_KV_E4M3) {   // the biased codes added 1152 * sum(q) to every score of a head
                    sc[nt][0] -= qbias[nt][0]; sc[nt][1] -= qbias[nt][1];
                    sc[nt][2] -= qbias[nt][0]; sc[nt][3] -= qbias[nt][1];
                }
                sc[nt][0] = dead0 ? -INFINITY : (sc[nt][0] + sd[nt][0]) * ks0;
                sc[nt][1] = dead0 ? -INFINITY : (sc[nt][1] + sd[nt][1]) * ks0;
                sc[nt][2] = dead1 ? -INFINITY : (sc[nt][2] + sd[nt][2]) * ks1;
                sc[nt][3] = dead1 ? -INFINITY : (sc[nt][3] + sd[nt][3]) * ks1;
#pragma unroll
                for (int j = 0; j < 2; ++j) {   // maximum over the 16 tokens: this lane's two rows, then the 8 lanes g
                    float mx = fmaxf(sc[nt][j], sc[nt][j + 2]);
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                    mnew[nt][j] = fmaxf(mrun[nt][j], mx);
                    grow |= mnew[nt][j] > mrun[nt][j];
                }
            }
            if (__any_sync(0xffffffffu, grow)) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const float c0 = fast_exp2(mrun[nt][0] - mnew[nt][0]), c1 = fast_exp2(mrun[nt][1] - mnew[nt][1]);
                    lrun[nt][0] *= c0;
                    lrun[nt][1] *= c1;
#pragma unroll
                    for (int c = 0; c < NCH; ++c) {
                        o[nt][c][0] *= c0; o[nt][c][1] *= c1;
                        o[nt][c][2] *= c0; o[nt][c][3] *= c1;
                    }
                    if (V_BIASED) {
                        psum[nt][0] *= c0; psum[nt][1] *= c1;
                        psum[nt][2] *= c0; psum[nt][3] *= c1;
                    }
                    mrun[nt][0] = mnew[nt][0];
                    mrun[nt][1] = mnew[nt][1];
                }
            }
            // P^T as the B operand of O^T = V^T P^T: the accumulator layout holds (token g | g+8, heads 2tq, 2tq+1);
            // a transposing 8x8 move turns it into (tokens 2tq, 2tq+1 | +8, head g)
            uint32_t pb[NT][2];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const float p0 = fast_exp2(sc[nt][0] - mrun[nt][0]), p1 = fast_exp2(sc[nt][1] - mrun[nt][1]);
                const float p2 = fast_exp2(sc[nt][2] - mrun[nt][0]), p3 = fast_exp2(sc[nt][3] - mrun[nt][1]);
                lrun[nt][0] += p0 + p2;
                lrun[nt][1] += p1 + p3;
                pb[nt][0] = movmatrix_trans(pack_half2(p0 * vs0, p1 * vs0));
                pb[nt][1] = movmatrix_trans(pack_half2(p2 * vs1, p3 * vs1));
            }

            // O^T += V^T P^T.  A transposed 8x8 b16 matrix hands lane (g, tq) the bytes
            // [v(t0,2g), v(t0,2g+1), v(t0+1,2g), v(t0+1,2g+1)], t0 = 2tq, of a 16-byte chunk: after the byte
            // shuffle the even channel 2g of both tokens is row g and the odd channel 2g+1 row g+8 of the M tile.
            if (V4) {
                // A transposed 8x8 b16 matrix of 4-bit codes hands lane (g, tq) the 16-bit words of tokens 2tq and
                // 2tq+1 that hold channels 4g..4g+3 of a 32-channel chunk: nibble i of both words, put into the
                // mantissa of 1024, is the A register (channel 4g+i, tokens 2tq | 2tq+1).  Rows g / g+8 of the M tile
                // are channels 4g, 4g+1 for accumulator 2c and 4g+2, 4g+3 for accumulator 2c+1 of chunk c.
#pragma unroll
                for (int m = 0; m < 2; ++m) {
                    uint32_t r[4];   // (tokens 0-7, chunk 2m), (tokens 8-15, chunk 2m), (0-7, 2m+1), (8-15, 2m+1)
                    ldsm_x4_t(v4base + ((v4ch + (uint32_t)(2 * m)) ^ v4sw) * 16, r[0], r[1], r[2], r[3]);
#pragma unroll
                    for (int cc = 0; cc < 2; ++cc) {
                        const uint32_t lo = r[2 * cc], hi = r[2 * cc + 1];   // tokens 0-7 | 8-15 of chunk 2m + cc
                        // nibbles 0 and 2 go into mantissa bits 0-3 (the number u + 1024), nibbles 1 and 3 stay in bits
                        // 4-7 (the number 16 u + 1024): no shift per nibble, and the factor 16 of the odd channels
                        // (rows g+8 of the M tile) is divided out of the accumulators at the end
                        const uint32_t lo8 = __byte_perm(lo, 0u, 0x4341), hi8 = __byte_perm(hi, 0u, 0x4341);   // >> 8 of both halves
                        uint32_t a0[4], a1[4];
                        a0[0] = and_or(lo, 0x000F000Fu, 0x64006400u);
                        a0[1] = and_or(lo, 0x00F000F0u, 0x64006400u);
                        a1[0] = and_or(lo8, 0x000F000Fu, 0x64006400u);
                        a1[1] = and_or(lo8, 0x00F000F0u, 0x64006400u);
                        a0[2] = and_or(hi, 0x000F000Fu, 0x64006400u);
                        a0[3] = and_or(hi, 0x00F000F0u, 0x64006400u);
                        a1[2] = and_or(hi8, 0x000F000Fu, 0x64006400u);
                        a1[3] = and_or(hi8, 0x00F000F0u, 0x64006400u);
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            mma_f16(o[nt][2 * (2 * m + cc)], a0, pb[nt][0], pb[nt][1]);
                            mma_f16(o[nt][2 * (2 * m + cc) + 1], a1, pb[nt][0], pb[nt][1]);
                        }
                    }
                }
            } else {
#pragma unroll
            for (int m = 0; m < NCH / 2; ++m) {
                uint32_t r0, r1, r2, r3;
                ldsm_x4_t(vbase + (((uint32_t)(2 * m) + ld_ch) ^ sw) * 16, r0, r1, r2, r3);
                uint32_t a0[4], a1[4];
                cvt_quad_v<KVT>(r0, a0[0], a0[1]);   // tokens 0-7:  even | odd channel
                cvt_quad_v<KVT>(r1, a0[2], a0[3]);   // tokens 8-15
                cvt_quad_v<KVT>(r2, a1[0], a1[1]);
                cvt_quad_v<KVT>(r3, a1[2], a1[3]);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    mma_f16(o[nt][2 * m], a0, pb[nt][0], pb[nt][1]);
                    mma_f16(o[nt][2 * m + 1], a1, pb[nt][0], pb[nt][1]);
                }
            }
            }
            if (V_BIASED) {   // sum_t p_t on the same path as O: a tile of ones in V's place
                const uint32_t ones[4] = {0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u};
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) mma_f16(psum[nt], ones, pb[nt][0], pb[nt][1]);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar + s * 8);
    }

    SKV_PHASE(4);
    SKV_CTA_STAMP(2);
    if (V4) {   // rows g hold u + 1024 = q + 1032, rows g+8 hold 16 u + 1024 = 16 (q + 72)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int c = 0; c < NCH; ++c)
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    o[nt][c][j] -= V4_BIAS * psum[nt][j];
                    o[nt][c][j + 2] = (o[nt][c][j + 2] - (1024.f + 16.f * 8.f) * psum[nt][j + 2]) * 0.0625f;
                }
    } else if (V_BIASED) {   // take the codes' bias out of O
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int c = 0; c < NCH; ++c)
#pragma unroll
                for (int j = 0; j < 4; ++j) o[nt][c][j] -= V_BIAS * psum[nt][j];
    }
    // the running sums are per lane (its two token rows): total over the 8 lanes g
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            lrun[nt][j] += __shfl_xor_sync(0xffffffffu, lrun[nt][j], 4);
            lrun[nt][j] += __shfl_xor_sync(0xffffffffu, lrun[nt][j], 8);
            lrun[nt][j] += __shfl_xor_sync(0xffffffffu, lrun[nt][j], 16);
        }

    named_bar_sync(1, Q8_CONSUMER_THREADS);
    float* mo = reinterpret_cast<float*>(smem);
    float* mm = mo + Q8_WARPS * MAX_GROUP * D;
    float* ml = mm + Q8_WARPS * MAX_GROUP;
    {
        float* my = mo + (warp * MAX_GROUP) * D;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int head = nt * 8 + tq * 2 + j;
                if (head < G) {
#pragma unroll
                    for (int c = 0; c < NCH; ++c) {
                        const int ch = V4 ? (c >> 1) * 32 + g * 4 + (c & 1) * 2 : c * 16 + g * 2;
                        *reinterpret_cast<float2*>(my + head * D + ch) = make_float2(o[nt][c][j], o[nt][c][j + 2]);
                    }
                    if (g == 0) { mm[warp * MAX_GROUP + head] = mrun[nt][j]; ml[warp * MAX_GROUP + head] = lrun[nt][j]; }
                }
            }
    }
    named_bar_sync(1, Q8_CONSUMER_THREADS);
    EpilogueArgs ea;
    ea.partial_o = p.partial_o; ea.partial_ml = p.partial_ml; ea.tickets = p.tickets; ea.out = p.out;
    ea.out_bf16 = p.out_bf16 != 0;
    ea.Hkv = p.Hkv; ea.G = G; ea.num_splits = p.num_splits; ea.o_stride_b = p.o_stride_b; ea.o_stride_h = p.o_stride_h;
    SKV_PHASE(5);
    merge_and_combine<D, Q8_WARPS, (NG == 1 ? 8 : 20)>(ea, smem, last_flag, b, h, split, n_splits, 1.f / P_BOOST);   // (the two-CTAs-per-SM variants have 128 registers)
    SKV_PHASE(6);
    SKV_PHASE_LAST_END();
    SKV_CTA_STAMP(3);
}

template <int KVT, int NT, int NG, bool V4 = false>
static int launch_q8(const CUtensorMap& tmK, const CUtensorMap& tmV, const Q8Params& p, int B, cudaStream_t stream) {
    static int configured_smem[64] = {0};
    const size_t smem = q8_smem_bytes<NG, V4>(p.stages);
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && configured_smem[dev] < (int)smem) {
        SKV_CUDA_TRY(cudaFuncSetAttribute(gqa_decode_q8_kernel<KVT, NT, NG, V4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured_smem[dev] = (int)smem;
    }
    const dim3 grid = p.list_items > 0 ? dim3(p.Hkv, p.list_items, 1) : dim3(p.Hkv, p.num_splits, B);
    SKV_CUDA_TRY(launch_pdl(gqa_decode_q8_kernel<KVT, NT, NG, V4>, grid, dim3(q8_threads(NG)), smem, stream, tmK, tmV, p));
    SKV_CUDA_TRY(cudaGetLastError());
    return SKV_OK;
}

}  // namespace gqa
}  // namespace skv

using namespace skv;

extern "C" {

#ifdef SKV_PROFILE_PHASES
int skv_debug_phase_ts_q8(unsigned long long* out) {
    return cudaMemcpyFromSymbol(out, skv_phase_ts, sizeof(unsigned long long) * 32) == cudaSuccess ? 0 : -4;
}
// per CTA (linear id < 1024): first instruction, first tile consumed, last tile consumed, exit; and the SM it ran on
int skv_debug_cta_ts_q8(unsigned long long* out) {
    return cudaMemcpyFromSymbol(out, skv::gqa::skv_cta_ts, sizeof(unsigned long long) * 5 * 1024) == cudaSuccess ? 0 : -4;
}
#endif

int skv_gqa_set_q8_stages(int stages) {
    // even, so that a stage is always drained by the same consumer group
    if (stages < 4 || stages > 12 || stages % 2) return fail(SKV_ERR_BAD_ARG, "q8 stages must be even and in 4..12: %d", stages);
    gqa::tuning().q8_stages = stages;
    return SKV_OK;
}

// FP8 caches with up to 8 query heads per kv-head: 1 forces the one-group kernel variant that fits two CTAs on an SM,
// 0 forces the two-group variant (one CTA per SM), -1 (default) lets the launcher choose by problem size.  Process-wide.
int skv_gqa_set_q8_two_per_sm(int mode) {
    if (mode < -1 || mode > 1) return fail(SKV_ERR_BAD_ARG, "mode must be -1, 0 or 1: %d", mode);
    gqa::tuning().q8_two_per_sm = mode;
    return SKV_OK;
}

// 1 (default): a ragged batch (seq_lens given) with few (sequence, kv-head) pairs is scheduled from a work list that
// every CTA derives from the real lengths (one wave of CTAs of nearly equal length); 0: always the host's static
// split plan.  Same results either way.  Process-wide.
int skv_gqa_set_ragged_worklist(int on) {
    if (on < 0 || on > 4) return fail(SKV_ERR_BAD_ARG, "work-list waves must be in 0..4: %d", on);
    gqa::tuning().ragged_worklist = on;   // values above 1: that many waves of proportionally shorter CTAs (experiments)
    return SKV_OK;
}

int skv_gqa_decode_paged(const void* q, const void* k_pool, const void* v_pool, const float* k_scale_pool,
                         const float* v_scale_pool, const int* page_table, const int* seq_lens, void* out,
                         void* workspace, size_t workspace_bytes, int B, int N, int Hq, int Hkv, int D, int kv_dtype,
                         int page_size, int max_pages, int num_pages, long long pool_stride_page,
                         long long pool_stride_head, long long pool_stride_slot, long long scale_stride_page,
                         long long scale_stride_head, float scale, int device, void* stream) {
    const int out_bf16 = (kv_dtype & SKV_OUT_BF16) ? 1 : 0;
    const bool v4 = (kv_dtype & SKV_V_INT4) != 0;
    const bool early_except_last = (kv_dtype & SKV_EARLY_EXCEPT_LAST) != 0;
    kv_dtype &= ~(SKV_OUT_BF16 | SKV_V_INT4 | SKV_EARLY_EXCEPT_LAST);
    if (!q || !k_pool || !v_pool || !k_scale_pool || !v_scale_pool || !out)
        return fail(SKV_ERR_BAD_ARG, "skv_gqa_decode_paged: null tensor pointer");
    if (B <= 0 || N <= 0 || Hq <= 0 || Hkv <= 0 || num_pages <= 0 || max_pages <= 0)
        return fail(SKV_ERR_BAD_ARG, "skv_gqa_decode_paged: sizes must be positive");
    if (Hq % Hkv != 0) return fail(SKV_ERR_BAD_ARG, "Hq=%d must be divisible by Hkv=%d", Hq, Hkv);
    const int G = Hq / Hkv;
    if (G > gqa::MAX_GROUP) return fail(SKV_ERR_UNSUPPORTED, "group size %d exceeds %d", G, gqa::MAX_GROUP);
    if (D != gqa::Q8_D) return fail(SKV_ERR_UNSUPPORTED, "8-bit KV decode supports head dim 128 only (got %d)", D);
    if (kv_dtype != SKV_KV_I8 && kv_dtype != SKV_KV_E4M3) return fail(SKV_ERR_UNSUPPORTED, "kv_dtype %d is not an 8-bit type", kv_dtype);
    if (page_size < gqa::CHUNK || page_size % gqa::CHUNK) return fail(SKV_ERR_UNSUPPORTED, "page_size %d must be a multiple of 16", page_size);
    if ((long long)max_pages * page_size < N) return fail(SKV_ERR_BAD_ARG, "max_pages * page_size < N");
    if (!(scale > 0.f)) return fail(SKV_ERR_BAD_ARG, "softmax scale must be positive");
    if ((scale_stride_page % 4) || (scale_stride_head % 4) || (reinterpret_cast<uintptr_t>(k_scale_pool) & 15) ||
        (reinterpret_cast<uintptr_t>(v_scale_pool) & 15))
        return fail(SKV_ERR_BAD_ARG, "scale pools must be 16-byte aligned with strides that are multiples of 4 floats");
    if (Hkv > 65535 || B > 65535) return fail(SKV_ERR_UNSUPPORTED, "grid dimension too large");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(SKV_ERR_CUDA, "cannot switch to device %d", device);

    // FP8 with up to 8 heads per group runs the one-group variant, two CTAs per SM: measured equal or faster at every
    // size tried (one sequence of 64K: equal; 4 x 64K: 0.76 -> 0.92 of the copy bandwidth; 16 x 64K: 0.89 -> 0.96).
    // INT8 takes it when the launch has more CTAs than one wave (16 x 64K: 0.87 -> 0.90); a single wave is faster
    // with two groups in one CTA per SM (one sequence of 64K: 34.9 against 37.9 us).
    const int two = gqa::tuning().q8_two_per_sm;   // -1: as above; 0 / 1: forced (experiments)
    const bool one_wave = seq_lens == nullptr && (long long)B * Hkv * 2 <= sm_count(device);
    const bool many = two >= 0 ? two != 0 : (kv_dtype == SKV_KV_E4M3 || !one_wave);
    const int slots = (G <= 8 && many) ? 2 : 1;   // CTAs resident per SM
    gqa::Plan pl = gqa::make_plan(B, N, Hq, Hkv, D, device, seq_lens != nullptr, slots);
    if (!workspace || workspace_bytes < pl.total)
        return fail(SKV_ERR_WORKSPACE, "workspace of %zu bytes is smaller than the %zu required", workspace_bytes, pl.total);
    if (reinterpret_cast<uintptr_t>(workspace) & 255) return fail(SKV_ERR_WORKSPACE, "workspace must be 256-byte aligned");

    // Pick how stages are fetched (see the Q8_* modes): fused page records when the four pools are views of one
    // [num_pages, Hkv, 33, 128]-byte buffer, 64-token boxes when pages allow it, 16-token chunks otherwise.
    const uint8_t* kb = static_cast<const uint8_t*>(k_pool);
    int mode = gqa::Q8_SEPARATE16;
    if (page_size == gqa::CHUNK && static_cast<const uint8_t*>(v_pool) == kb + 16 * D &&
        reinterpret_cast<const uint8_t*>(k_scale_pool) == kb + 32 * D &&
        reinterpret_cast<const uint8_t*>(v_scale_pool) == kb + 32 * D + 64 && pool_stride_slot == D &&
        pool_stride_head == gqa::RECORD_BYTES && pool_stride_page == (long long)Hkv * gqa::RECORD_BYTES &&
        scale_stride_head * 4 == pool_stride_head && scale_stride_page * 4 == pool_stride_page)
        mode = gqa::Q8_FUSED;
    else if (page_size % gqa::TILE == 0)
        mode = gqa::Q8_SEPARATE64;

    if (v4) {
        // K in 8 bits, V in 4: only as mixed-precision page records, [num_pages, Hkv, 25, 128] bytes
        if (G > 8) return fail(SKV_ERR_UNSUPPORTED, "4-bit V pages serve up to 8 query heads per kv-head (got %d)", G);
        if (!(page_size == gqa::CHUNK && static_cast<const uint8_t*>(v_pool) == kb + 16 * D &&
              reinterpret_cast<const uint8_t*>(k_scale_pool) == kb + 24 * D &&
              reinterpret_cast<const uint8_t*>(v_scale_pool) == kb + 24 * D + 64 && pool_stride_slot == D &&
              pool_stride_head == gqa::V4_RECORD_BYTES && pool_stride_page == (long long)Hkv * gqa::V4_RECORD_BYTES &&
              scale_stride_head * 4 == pool_stride_head && scale_stride_page * 4 == pool_stride_page))
            return fail(SKV_ERR_UNSUPPORTED, "SKV_V_INT4 needs the four pools to be views of one [num_pages, Hkv, 25, 128]-byte "
                                             "buffer of mixed-precision page records (16-token pages)");
        mode = gqa::Q8_FUSED;
    }

    CUtensorMap tmK, tmV;
    PoolMapPos pos, pos2;
    int rc;
    if (v4) {
        rc = make_pool_tmap(&tmK, &pos, k_pool, D, num_pages, Hkv, gqa::V4_RECORD_ROWS, pool_stride_page, pool_stride_head,
                            pool_stride_slot, gqa::V4_RECORD_ROWS);
        if (rc) return rc;
        tmV = tmK;
    } else if (mode == gqa::Q8_FUSED) {
        rc = make_pool_tmap(&tmK, &pos, k_pool, D, num_pages, Hkv, gqa::RECORD_ROWS, pool_stride_page, pool_stride_head,
                            pool_stride_slot, gqa::RECORD_ROWS);
        if (rc) return rc;
        tmV = tmK;
    } else {
        const int box = mode == gqa::Q8_SEPARATE64 ? gqa::TILE : gqa::CHUNK;
        rc = make_pool_tmap(&tmK, &pos, k_pool, D, num_pages, Hkv, page_size, pool_stride_page, pool_stride_head,
                            pool_stride_slot, box);
        if (rc) return rc;
        rc = make_pool_tmap(&tmV, &pos2, v_pool, D, num_pages, Hkv, page_size, pool_stride_page, pool_stride_head,
                            pool_stride_slot, box);
        if (rc) return rc;
    }

    gqa::Q8Params p;
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    p.q = static_cast<const __half*>(q);
    p.out = static_cast<__half*>(out);
    p.tickets = reinterpret_cast<int*>(ws + pl.off_tickets);
    p.status = reinterpret_cast<int*>(ws + pl.off_status);
    p.partial_ml = reinterpret_cast<float*>(ws + pl.off_ml);
    p.partial_o = reinterpret_cast<float*>(ws + pl.off_o);
    p.seq_lens = seq_lens;
    p.page_table = page_table;
    p.k_scale = k_scale_pool;
    p.v_scale = v_scale_pool;
    p.N = N; p.Hq = Hq; p.Hkv = Hkv; p.G = G;
    p.tiles_per_split = pl.tiles_per_split;
    p.num_splits = pl.splits;
    // two CTAs per SM share the shared memory: at most 6 stages each, 4 when the launch is a single wave of CTAs
    // (a shorter ring fills sooner, which is what a short-lived CTA notices)
    const int cap2 = one_wave ? 4 : 6;
    p.stages = slots == 2 ? (gqa::tuning().q8_stages < cap2 ? gqa::tuning().q8_stages : cap2) : gqa::tuning().q8_stages;
    p.out_bf16 = out_bf16;
    p.early_kv = early_except_last ? 2 : gqa::tuning().early_kv;
    p.page_size = page_size;
    p.max_pages = max_pages;
    p.num_pages = num_pages;
    // work-list mode: ragged lengths, few pairs (a quarter of the resident CTA slots at most), a short batch to walk
    const int slots_total = sm_count(device) * slots;
    // (measured at 16 ragged sequences: 1 kv-head 0.60 -> 0.77 of the copy bandwidth, 2 kv-heads 0.75 -> 0.86, 4 kv-heads
    // 0.88 -> 0.84: the static plan is kept from a quarter of the slots up)
    const int waves = gqa::tuning().ragged_worklist;
    const bool worklist = seq_lens != nullptr && waves > 0 && B <= 64 && (long long)B * Hkv * 8 <= slots_total;
    p.list_items = worklist ? slots_total * waves / Hkv : 0;
    p.B = B;
    p.mode = mode;
    p.sc_sp = scale_stride_page; p.sc_sh = scale_stride_head;
    p.q_stride_b = (long long)Hq * D; p.q_stride_h = D;
    p.o_stride_b = (long long)Hq * D; p.o_stride_h = D;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.pos = pos;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (v4) {
        if (slots == 2)
            return kv_dtype == SKV_KV_E4M3 ? gqa::launch_q8<SKV_KV_E4M3, 1, 1, true>(tmK, tmV, p, B, st)
                                           : gqa::launch_q8<SKV_KV_I8, 1, 1, true>(tmK, tmV, p, B, st);
        return kv_dtype == SKV_KV_E4M3 ? gqa::launch_q8<SKV_KV_E4M3, 1, 2, true>(tmK, tmV, p, B, st)
                                       : gqa::launch_q8<SKV_KV_I8, 1, 2, true>(tmK, tmV, p, B, st);
    }
    if (slots == 2)
        return kv_dtype == SKV_KV_E4M3 ? gqa::launch_q8<SKV_KV_E4M3, 1, 1>(tmK, tmV, p, B, st)
                                       : gqa::launch_q8<SKV_KV_I8, 1, 1>(tmK, tmV, p, B, st);
    if (G <= 8)
        return kv_dtype == SKV_KV_E4M3 ? gqa::launch_q8<SKV_KV_E4M3, 1, 2>(tmK, tmV, p, B, st)
                                       : gqa::launch_q8<SKV_KV_I8, 1, 2>(tmK, tmV, p, B, st);
    return kv_dtype == SKV_KV_E4M3 ? gqa::launch_q8<SKV_KV_E4M3, 2, 2>(tmK, tmV, p, B, st)
                                   : gqa::launch_q8<SKV_KV_I8, 2, 2>(tmK, tmV, p, B, st);
}

}  // extern "C"
