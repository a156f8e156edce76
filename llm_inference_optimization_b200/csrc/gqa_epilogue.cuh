// Shared by the dense decode kernels (fp16 and 8-bit KV): tile geometry, the
// split plan and workspace layout, and the epilogue that merges the consumer
// warps of a CTA, publishes the split partial and lets the last CTA of each
// (batch, kv-head) do the log-sum-exp combine.
//
// No reference counterpart: the reference kernel never splits the KV length
// (csrc/kernels/gqa_decode.cu:255 launches one CTA per query head).
#pragma once

#include <cuda_bf16.h>

#include "skv_common.cuh"

namespace skv {
namespace gqa {

constexpr int TILE = 64;            // tokens per pipeline stage
constexpr int CONSUMER_WARPS = 4;   // fp16 kernel: each warp takes TILE / 4 = 16 tokens of a stage
constexpr int CONSUMER_THREADS = CONSUMER_WARPS * 32;
constexpr int THREADS = CONSUMER_THREADS + 32;
constexpr int MAX_CONSUMER_WARPS = 12;  // the 8-bit kernel runs up to three groups of four warps on rotating stages
constexpr int MAX_SPLITS = 512;
constexpr int MAX_GROUP = 16;       // query heads per kv head (rows of one MMA tile)

// Shared-memory words the epilogue needs at the start of the (drained) stage ring.
template <int D, int NW = CONSUMER_WARPS>
__host__ __device__ constexpr size_t merge_smem_bytes() {
    return (size_t)NW * MAX_GROUP * D * 4 + (size_t)NW * MAX_GROUP * 8 + (size_t)NW * MAX_SPLITS * 4;
}

// Short contexts: the splits of one (batch, kv-head) form a thread-block cluster and the split results are summed
// through distributed shared memory instead of a global-memory round trip (merge_and_combine_cluster).
constexpr int MAX_CLUSTER_SPLITS = 16;
// Each CTA's merged result for that sum: O [MAX_GROUP][D] and (max, sum) [MAX_GROUP][2], behind the merge area.
template <int D, int NW = CONSUMER_WARPS>
__host__ __device__ constexpr size_t cluster_area_offset() {
    return (merge_smem_bytes<D, NW>() + 15) & ~size_t(15);
}
template <int D, int NW = CONSUMER_WARPS>
__host__ __device__ constexpr size_t epilogue_smem_bytes() {
    return cluster_area_offset<D, NW>() + (size_t)MAX_GROUP * D * 4 + (size_t)MAX_GROUP * 8;
}

struct Tuning {
    int stages = 4;        // fp16 ring depth (64-token stages of 32 KB at D = 128)
    int ctas_per_sm = 1;
    int q8_stages = 8;     // 8-bit ring depth (stages of 17 KB)
    int early_kv = 0;      // 1: K/V, page table and lengths may be read before the previous kernel has completed
    int q8_two_per_sm = -1;  // FP8 kernel variant: -1 chosen by the launcher, 0 one CTA per SM, 1 two CTAs per SM
    int ragged_worklist = 1;  // the 8-bit kernel schedules a ragged batch with few pairs from a device-side work list
    int cluster_combine = 1;  // short contexts: splits of a (batch, kv-head) as one cluster, summed through shared memory
};
inline Tuning& tuning() {
    static Tuning t;
    return t;
}

// Fewest 64-token tiles a split may hold: shorter CTAs are dominated by their start and end.
#ifndef SKV_MIN_TILES_PER_SPLIT
#define SKV_MIN_TILES_PER_SPLIT 16
#endif

// Waves of CTAs the KV length is cut into when the per-sequence lengths are not known to the host.
#ifndef SKV_RAGGED_WAVES
#define SKV_RAGGED_WAVES 8
#endif

constexpr size_t WORKSPACE_HEAD_BYTES = 65536;   // status word + tickets, at the same place for every problem size

struct Plan {
    int splits, tiles_per_split;
    size_t off_status, off_tickets, off_ml, off_o, total;
};

// How the KV length is cut into whole 64-token tiles per split: one CTA per SM (times ctas_per_sm) when
// there are few (batch, kv-head) pairs, about four waves of CTAs when there are many.
inline Plan make_plan(int B, int N, int Hq, int Hkv, int D, int device, bool ragged = false, int slots_per_sm = 0) {
    Plan pl;
    const int G = Hq / Hkv;
    const long long total_tiles = (N + TILE - 1) / TILE;
    const long long pairs = (long long)B * Hkv;
    const long long target = (long long)sm_count(device) * (slots_per_sm > 0 ? slots_per_sm : tuning().ctas_per_sm);
    long long splits;
    if (!ragged && pairs * 2 <= target) {
        splits = target / pairs;              // few equally long (batch, head) pairs: one wave, one CTA per SM
    } else {
        // Many pairs, or per-sequence lengths the host does not know: a CTA streams at about 1/SMs of the HBM
        // rate, so work is cut into about eight waves of CTAs to let long sequences spread over many SMs
        // (CTAs past a sequence's end exit at once).
        const long long max_by_size = total_tiles / SKV_MIN_TILES_PER_SPLIT > 0 ? total_tiles / SKV_MIN_TILES_PER_SPLIT : 1;
        if (ragged) {
            splits = (SKV_RAGGED_WAVES * target + pairs - 1) / pairs;
        } else {
            // equal lengths: every CTA lasts the same, so pick the split count between about 2 and 8 waves whose
            // last wave is fullest (pairs * splits CTAs over `target` slots), the smallest such count on ties
            splits = 1;
            double best = 0.0;
            const long long lo = (2 * target + pairs - 1) / pairs, hi = (8 * target + pairs - 1) / pairs;
            for (long long c = lo < 1 ? 1 : lo; c <= hi && c <= max_by_size; ++c) {
                const double w = (double)(pairs * c) / (double)target;
                const double eff = w / (double)(long long)(w + 0.999999);
                if (eff > best + 0.02) { best = eff; splits = c; }
            }
        }
        if (splits > max_by_size) splits = max_by_size;
    }
    if (splits < 1) splits = 1;
    if (splits > total_tiles) splits = total_tiles;
    if (splits > MAX_SPLITS) splits = MAX_SPLITS;
    long long tps = (total_tiles + splits - 1) / splits;
    splits = (total_tiles + tps - 1) / tps;
    pl.splits = (int)splits;
    pl.tiles_per_split = (int)tps;
    auto up = [](size_t x) { return (x + 255) & ~size_t(255); };
    // The device status word sits at offset 0 of every workspace and the tickets (which must be zero when a launch
    // starts, and are left zero by it) behind it, in a head region whose size does not depend on the problem: a
    // later call with more (batch, kv-head) pairs must not find an earlier call's partial sums where its tickets
    // live.  Beyond 16320 pairs the region grows with the problem and such a workspace must be cleared before it
    // is reused with more pairs.
    size_t off = 256;
    pl.off_status = 0;
    pl.off_tickets = off;
    off += up((size_t)B * Hkv * sizeof(int));
    if (off < WORKSPACE_HEAD_BYTES) off = WORKSPACE_HEAD_BYTES;
    pl.off_ml = off;
    off += up((size_t)B * Hkv * splits * G * 2 * sizeof(float));
    pl.off_o = off;
    off += up((size_t)B * Hkv * splits * G * D * sizeof(float));
    pl.total = off;
    return pl;
}

#if defined(__CUDACC__)

// Work-list schedule of a ragged batch with few (sequence, kv-head) pairs.  The host cannot read seq_lens, so its
// plan cuts the LONGEST possible sequence into many short splits and launches that many CTAs for every sequence:
// short splits each pay a pipeline fill, a merge and a partial, and the CTAs past a sequence's end are launched only
// to exit (measured at 16 sequences x 1 kv-head: 0.60 of the copy bandwidth against 0.83 for the same bytes with
// lengths the host knows).  In this mode the grid is (Hkv, list_items): every CTA adds up the real lengths, sizes
// the splits so that all (sequence, split) items of a kv-head fit the list_items CTAs launched for it -- one wave of
// CTAs of nearly equal length -- and finds its own item by a prefix walk over the sequences (B <= 64).
struct SplitItem {
    int b, split, len, n_splits, tiles_per_split;   // b < 0: past the end of the work list
};

__device__ __forceinline__ SplitItem worklist_item(const int* seq_lens, int B, int N, int list_items, int item,
                                                   int host_tiles_per_split) {
    long long tiles = 0;
    for (int i = 0; i < B; ++i) tiles += (min(max(seq_lens[i], 0), N) + TILE - 1) / TILE;
    const long long room = max(1, list_items - B);   // every sequence may add one partial split
    SplitItem it;
    // never shorter than the host's splits: the partial arrays are sized for the host's split count
    it.tiles_per_split = max(host_tiles_per_split, (int)((tiles + room - 1) / room));
    it.b = -1;
    it.split = 0;
    it.len = 0;
    it.n_splits = 1;
    int acc = 0;
    for (int i = 0; i < B; ++i) {
        const int li = min(max(seq_lens[i], 0), N);
        const int ti = (li + TILE - 1) / TILE;
        const int ns = ti > 0 ? (ti + it.tiles_per_split - 1) / it.tiles_per_split : 1;   // an empty sequence still writes zeros
        if (it.b < 0 && item < acc + ns) { it.b = i; it.split = item - acc; it.len = li; it.n_splits = ns; }
        acc += ns;
    }
    return it;
}

struct EpilogueArgs {
    float* partial_o;    // [B, Hkv, S, G, D]
    float* partial_ml;   // [B, Hkv, S, G, 2]
    int* tickets;        // [B * Hkv]
    __half* out;         // element (b, hq, d) at b*o_stride_b + hq*o_stride_h + d
    int Hkv, G, num_splits;
    long long o_stride_b, o_stride_h;
    bool out_bf16 = false;   // store bf16 instead of fp16 (same element size and strides)
    float* ml_final = nullptr;  // optional [B, Hkv * G, 2]: softmax maximum (exp2 domain) and denominator of every head
};

__device__ __forceinline__ uint16_t out_bits(float x, bool bf16) {
    return bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(x)) : __half_as_ushort(__float2half_rn(x));
}

// Called by all NW * 32 consumer threads (threadIdx.x < NW * 32) after every
// warp has stored its state at `smem`: O [NW][MAX_GROUP][D], running max
// [NW][MAX_GROUP] (exp2 domain), running sum [NW][MAX_GROUP], and after a named
// barrier.  `out_scale` multiplies the un-normalised output (1 for fp16 KV).
template <int D, int NW = CONSUMER_WARPS, int CB = 24>   // CB: partial rows in flight per lane in the last CTA's combine
__device__ __forceinline__ void merge_and_combine(const EpilogueArgs& p, uint8_t* smem, int* last_flag, int b, int h,
                                                  int split, int n_splits, float out_scale) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = p.G;
    float* mo = reinterpret_cast<float*>(smem);
    float* mm = mo + NW * MAX_GROUP * D;
    float* ml = mm + NW * MAX_GROUP;
    float* wts = ml + NW * MAX_GROUP;  // [W][MAX_SPLITS]

    const long long bh = (long long)b * p.Hkv + h;
    const long long pbase = (bh * p.num_splits + split) * G;  // row index into the partials
    for (int idx = threadIdx.x; idx < G * D; idx += (NW * 32)) {
        const int r = idx / D, d = idx - r * D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; ++w) M = fmaxf(M, mm[w * MAX_GROUP + r]);
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            const float mw = mm[w * MAX_GROUP + r];
            const float wgt = (mw == -INFINITY) ? 0.f : fast_exp2(mw - M);
            L += ml[w * MAX_GROUP + r] * wgt;
            O += mo[(w * MAX_GROUP + r) * D + d] * wgt;
        }
        O *= out_scale;
        if (n_splits == 1) {
            if (p.ml_final && d == 0) {
                p.ml_final[(bh * G + r) * 2] = M;
                p.ml_final[(bh * G + r) * 2 + 1] = L;
            }
            const float inv = L > 0.f ? 1.f / L : 0.f;
            reinterpret_cast<uint16_t*>(p.out)[(long long)b * p.o_stride_b + (long long)(h * G + r) * p.o_stride_h + d] =
                out_bits(O * inv, p.out_bf16);
        } else {
            p.partial_o[(pbase + r) * D + d] = O;
            if (d == 0) {
                p.partial_ml[(pbase + r) * 2 + 0] = M;
                p.partial_ml[(pbase + r) * 2 + 1] = L;
            }
        }
    }
    if (n_splits == 1) return;

    // ------------------------------------------- last CTA of this (b, h) combines
    __threadfence();
    named_bar_sync(1, (NW * 32));
    if (threadIdx.x == 0) {
        const int ticket = atomicAdd(&p.tickets[bh], 1);
        const int last = (ticket == n_splits - 1);
        if (last) p.tickets[bh] = 0;  // ready for the next launch on this workspace
        *last_flag = last;
    }
    named_bar_sync(1, (NW * 32));
    if (!*last_flag) return;
    __threadfence();

    // One warp per query head.  The partial rows do not depend on the weights, so the first CB of them are on their
    // way before the (max, sum) pairs are even read, and those pairs are read once and kept in registers: a combine
    // of up to CB splits costs one round trip to L2 where a weights-first order costs three or more, and it sits on
    // the critical path of every split launch.  Splits past the end read a real (clamped) row with weight zero, so
    // no load waits on a condition.  The sums run over the splits in ascending order, as before.
    const long long rbase = bh * p.num_splits * G;
    float* wrow = wts + warp * MAX_SPLITS;
    constexpr int MLR = 4;    // (max, sum) pairs per lane kept in registers: splits lane, lane + 32, ...
    const bool ol = lane < D / 4;
    const long long sstride = (long long)G * D;
    for (int r = warp; r < G; r += NW) {
        const float* src = p.partial_o + (rbase + r) * D + (ol ? lane * 4 : 0);
        float4 vo[CB];
#pragma unroll
        for (int j = 0; j < CB; ++j) vo[j] = __ldcg(reinterpret_cast<const float4*>(src + (long long)min(j, n_splits - 1) * sstride));
        float2 mlv[MLR];
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < MLR; ++i) {
            const int sidx = lane + 32 * i;
            mlv[i] = __ldcg(reinterpret_cast<const float2*>(&p.partial_ml[(rbase + (long long)min(sidx, n_splits - 1) * G + r) * 2]));
            if (sidx >= n_splits) mlv[i] = make_float2(-INFINITY, 0.f);
            mx = fmaxf(mx, mlv[i].x);
        }
        for (int sidx = lane + 32 * MLR; sidx < n_splits; sidx += 32) mx = fmaxf(mx, __ldcg(&p.partial_ml[(rbase + (long long)sidx * G + r) * 2]));
        mx = warp_max(mx);
        float Ls = 0.f;
#pragma unroll
        for (int i = 0; i < MLR; ++i) {
            const int sidx = lane + 32 * i;
            if (sidx < n_splits) {
                const float w = (mlv[i].x == -INFINITY) ? 0.f : fast_exp2(mlv[i].x - mx);
                Ls += mlv[i].y * w;
                wrow[sidx] = w;
            }
        }
        for (int sidx = lane + 32 * MLR; sidx < n_splits; sidx += 32) {
            const float2 v = __ldcg(reinterpret_cast<const float2*>(&p.partial_ml[(rbase + (long long)sidx * G + r) * 2]));
            const float w = (v.x == -INFINITY) ? 0.f : fast_exp2(v.x - mx);
            Ls += v.y * w;
            wrow[sidx] = w;
        }
        Ls = warp_sum(Ls);
        if (p.ml_final && lane == 0) {
            p.ml_final[(bh * G + r) * 2] = mx;
            p.ml_final[(bh * G + r) * 2 + 1] = Ls;
        }
        __syncwarp();
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s0 = 0; s0 < n_splits; s0 += CB) {
            if (s0) {
#pragma unroll
                for (int j = 0; j < CB; ++j) vo[j] = __ldcg(reinterpret_cast<const float4*>(src + (long long)min(s0 + j, n_splits - 1) * sstride));
            }
#pragma unroll
            for (int j = 0; j < CB; ++j) {
                const float w = s0 + j < n_splits ? wrow[s0 + j] : 0.f;
                acc.x += vo[j].x * w; acc.y += vo[j].y * w; acc.z += vo[j].z * w; acc.w += vo[j].w * w;
            }
        }
        if (ol) {
            const float inv = Ls > 0.f ? 1.f / Ls : 0.f;
            uint2 pk;
            pk.x = (uint32_t)out_bits(acc.x * inv, p.out_bf16) | ((uint32_t)out_bits(acc.y * inv, p.out_bf16) << 16);
            pk.y = (uint32_t)out_bits(acc.z * inv, p.out_bf16) | ((uint32_t)out_bits(acc.w * inv, p.out_bf16) << 16);
            *reinterpret_cast<uint2*>(p.out + (long long)b * p.o_stride_b + (long long)(h * G + r) * p.o_stride_h + lane * 4) = pk;
        }
        __syncwarp();
    }
}

// The cluster variant of merge_and_combine, for a launch whose clusters hold all splits of one (batch, kv-head) with
// cluster rank == split.  Called by the consumer threads of a CTA that has a split, after the same preparation as
// merge_and_combine; the caller then runs the two cluster barriers with EVERY thread of the cluster:
//     cluster_merge_publish (consumers)  ->  cluster_barrier (all)  ->  cluster_combine_rank0 (consumers of rank 0)
//     ->  cluster_barrier (all: no CTA leaves while rank 0 may still read its shared memory)
template <int D, int NW = CONSUMER_WARPS>
__device__ __forceinline__ void cluster_merge_publish(uint8_t* smem, int G, float out_scale) {
    float* mo = reinterpret_cast<float*>(smem);
    float* mm = mo + NW * MAX_GROUP * D;
    float* ml = mm + NW * MAX_GROUP;
    float* co = reinterpret_cast<float*>(smem + cluster_area_offset<D, NW>());   // [MAX_GROUP][D]
    float* cml = co + MAX_GROUP * D;                                             // [MAX_GROUP][2]
    for (int idx = threadIdx.x; idx < G * D; idx += (NW * 32)) {
        const int r = idx / D, d = idx - r * D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; ++w) M = fmaxf(M, mm[w * MAX_GROUP + r]);
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            const float mw = mm[w * MAX_GROUP + r];
            const float wgt = (mw == -INFINITY) ? 0.f : fast_exp2(mw - M);
            L += ml[w * MAX_GROUP + r] * wgt;
            O += mo[(w * MAX_GROUP + r) * D + d] * wgt;
        }
        co[idx] = O * out_scale;
        if (d == 0) {
            cml[2 * r] = M;
            cml[2 * r + 1] = L;
        }
    }
}

template <int D, int NW = CONSUMER_WARPS>
__device__ __forceinline__ void cluster_combine_rank0(const EpilogueArgs& p, uint8_t* smem, int b, int h, int n_splits) {
    const int G = p.G;
    const uint32_t co = smem_u32(smem + cluster_area_offset<D, NW>());
    const uint32_t cml = co + MAX_GROUP * D * 4;
    const long long bh = (long long)b * p.Hkv + h;
    for (int i4 = threadIdx.x; i4 < G * D / 4; i4 += (NW * 32)) {
        const int r = (i4 * 4) / D, d = i4 * 4 - r * D;
        // every remote load is issued before the first use (ranks past the last split read a real CTA's area, clamped,
        // and weigh zero): one trip through the cluster's shared memory instead of one per dependent step
        float2 mlv[MAX_CLUSTER_SPLITS];
        float4 ov[MAX_CLUSTER_SPLITS];
#pragma unroll
        for (int s = 0; s < MAX_CLUSTER_SPLITS; ++s) {
            const int rank = min(s, n_splits - 1);
            mlv[s] = ld_cluster_f2(cluster_map(cml + r * 8, rank));
            ov[s] = ld_cluster_f4(cluster_map(co + i4 * 16, rank));
        }
        float mx = -INFINITY;
#pragma unroll
        for (int s = 0; s < MAX_CLUSTER_SPLITS; ++s) {
            if (s >= n_splits) mlv[s] = make_float2(-INFINITY, 0.f);
            mx = fmaxf(mx, mlv[s].x);
        }
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        float Ls = 0.f;
#pragma unroll
        for (int s = 0; s < MAX_CLUSTER_SPLITS; ++s) {   // in split order: the sum does not depend on timing
            const float w = (mlv[s].x == -INFINITY) ? 0.f : fast_exp2(mlv[s].x - mx);
            Ls += mlv[s].y * w;
            acc.x += ov[s].x * w; acc.y += ov[s].y * w; acc.z += ov[s].z * w; acc.w += ov[s].w * w;
        }
        if (p.ml_final && d == 0) {
            p.ml_final[(bh * G + r) * 2] = mx;
            p.ml_final[(bh * G + r) * 2 + 1] = Ls;
        }
        const float inv = Ls > 0.f ? 1.f / Ls : 0.f;
        uint2 pk;
        pk.x = (uint32_t)out_bits(acc.x * inv, p.out_bf16) | ((uint32_t)out_bits(acc.y * inv, p.out_bf16) << 16);
        pk.y = (uint32_t)out_bits(acc.z * inv, p.out_bf16) | ((uint32_t)out_bits(acc.w * inv, p.out_bf16) << 16);
        *reinterpret_cast<uint2*>(p.out + (long long)b * p.o_stride_b + (long long)(h * G + r) * p.o_stride_h + d) = pk;
    }
}

#endif  // __CUDACC__

}  // namespace gqa
}  // namespace skv
