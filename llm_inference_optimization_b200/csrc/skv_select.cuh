// Exact top-k selection by one CTA: radix select on order-preserving keys, then
// an ordered compaction, so the chosen positions come out sorted ascending and
// equal scores resolve to the lower position.
//
// The reference selects with a per-thread one-slot "heap" merged by a single
// thread (csrc/kernels/kv_evict_quant.cu:181-239), which drops true top-k
// members, and with a serial min-replace loop on thread 0
// (csrc/kernels/sparse_attention.cu:88-117).  Both are replaced by this routine;
// its result equals torch.topk(...).indices as a set.
#pragma once

#include "skv_common.cuh"

namespace skv {

// Larger float <=> larger key (total order; -0 < +0, NaNs at the ends).
__device__ __forceinline__ uint32_t score_key(float f) {
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Shared-memory words block_topk_sorted needs for a CTA of NT threads.
template <int NT>
struct TopkSmem {
    static constexpr int NW = NT / 32;
    static constexpr int WORDS = NW * 256 + 4 * NW + 8;
};

// Writes the positions of the k largest of sc[0..T) to out[0..k), ascending.
// All NT threads of the CTA must call it; `sm` is TopkSmem<NT>::WORDS words.
// `sc` may live in global or shared memory and must not change during the call.
template <int NT>
__device__ void block_topk_sorted(const float* sc, int T, int k, int* out, uint32_t* sm) {
    constexpr int NW = NT / 32;
    constexpr int LOADS = 8;  // scores fetched per thread before any is processed
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (k <= 0) return;
    if (k >= T) {
        for (int i = tid; i < T; i += NT) out[i] = i;
        return;
    }
    uint32_t* hist = sm;                  // [NW][256]
    uint32_t* wcnt = sm + NW * 256;       // [4][NW]: gt, eq, sel-prefix, eq-prefix
    uint32_t* bc = wcnt + 4 * NW;         // broadcast: digit, remaining

    uint32_t prefix = 0, mask = 0;
    int remaining = k;
#pragma unroll 1
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        for (int i = tid; i < NW * 256; i += NT) hist[i] = 0;
        __syncthreads();
        uint32_t* myh = hist + warp * 256;
        for (int base = 0; base < T; base += NT * LOADS) {  // uniform trip count: the warp votes need every lane
            float v[LOADS];
#pragma unroll
            for (int u = 0; u < LOADS; ++u) {  // independent loads first: their latencies overlap
                const int i = base + u * NT + tid;
                v[u] = i < T ? sc[i] : 0.f;
            }
#pragma unroll
            for (int u = 0; u < LOADS; ++u) {
                const int i = base + u * NT + tid;
                const uint32_t key = score_key(v[u]);
                const bool act = i < T && (key & mask) == prefix;
                const uint32_t digit = (key >> shift) & 255u;
                // Scores cluster in a few exponent values, so the leading digits of a warp's 32 keys are often
                // all equal: then one lane adds the whole count instead of 32 conflicting atomics on one address.
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
        }
        __syncthreads();
        for (int b = tid; b < 256; b += NT) {  // fold the per-warp histograms into row 0
            uint32_t s = 0;
#pragma unroll 4
            for (int w = 0; w < NW; ++w) s += hist[w * 256 + b];
            hist[b] = s;
        }
        __syncthreads();
        if (warp == 0) {
            // lane l owns digits 255-8l .. 248-8l (descending); find where the running count reaches `remaining`
            uint32_t mine = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) mine += hist[255 - 8 * lane - j];
            uint32_t incl = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            const uint32_t hit = __ballot_sync(0xffffffffu, incl >= (uint32_t)remaining);
            const int owner = __ffs(hit) - 1;  // always found: matching keys >= remaining
            if (lane == owner) {
                uint32_t above = incl - mine;  // keys with a larger digit
                int d = 255 - 8 * lane;
                for (int j = 0; j < 8; ++j, --d) {
                    const uint32_t c = hist[d];
                    if (above + c >= (uint32_t)remaining) break;
                    above += c;
                }
                bc[0] = (uint32_t)d;
                bc[1] = (uint32_t)remaining - above;
            }
        }
        __syncthreads();
        prefix |= bc[0] << shift;
        mask |= 0xFFu << shift;
        remaining = (int)bc[1];
        __syncthreads();
    }
    const uint32_t thr = prefix;  // key of the k-th largest score
    const int need = remaining;   // how many scores equal to it are taken (lowest positions first)

    // contiguous, 32-aligned segment per warp
    int seg = (T + NW - 1) / NW;
    seg = (seg + 31) & ~31;
    const int s0 = min(T, warp * seg), s1 = min(T, s0 + seg);
    uint32_t gt = 0, eq = 0;
    for (int i0 = s0; i0 < s1; i0 += 32 * LOADS) {
        float v[LOADS];
#pragma unroll
        for (int u = 0; u < LOADS; ++u) {
            const int i = i0 + u * 32 + lane;
            v[u] = i < s1 ? sc[i] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < LOADS; ++u) {
            const bool in = i0 + u * 32 + lane < s1;
            const uint32_t key = score_key(v[u]);
            gt += __popc(__ballot_sync(0xffffffffu, in && key > thr));
            eq += __popc(__ballot_sync(0xffffffffu, in && key == thr));
        }
    }
    if (lane == 0) { wcnt[warp] = gt; wcnt[NW + warp] = eq; }
    __syncthreads();
    if (warp == 0) {
        uint32_t eqp = 0, selp = 0;
        for (int base = 0; base < NW; base += 32) {
            const int w = base + lane;
            const uint32_t g = w < NW ? wcnt[w] : 0u, e = w < NW ? wcnt[NW + w] : 0u;
            uint32_t ei = e;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t v = __shfl_up_sync(0xffffffffu, ei, o);
                if (lane >= o) ei += v;
            }
            const uint32_t eex = eqp + ei - e;  // ties before this warp's segment
            const uint32_t take = (uint32_t)max(0, min((int)e, need - (int)eex));
            const uint32_t s = g + take;
            uint32_t si = s;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t v = __shfl_up_sync(0xffffffffu, si, o);
                if (lane >= o) si += v;
            }
            if (w < NW) { wcnt[2 * NW + w] = selp + si - s; wcnt[3 * NW + w] = eex; }
            eqp += __shfl_sync(0xffffffffu, ei, 31);
            selp += __shfl_sync(0xffffffffu, si, 31);
        }
    }
    __syncthreads();
    uint32_t pos = wcnt[2 * NW + warp], eqrun = wcnt[3 * NW + warp];
    const uint32_t lt = (1u << lane) - 1u;
    for (int i0 = s0; i0 < s1; i0 += 32 * LOADS) {
        float v[LOADS];
#pragma unroll
        for (int u = 0; u < LOADS; ++u) {
            const int i = i0 + u * 32 + lane;
            v[u] = i < s1 ? sc[i] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < LOADS; ++u) {
            const int i = i0 + u * 32 + lane;
            const bool in = i < s1;
            const uint32_t key = score_key(v[u]);
            const bool isgt = in && key > thr, iseq = in && key == thr;
            const uint32_t beq = __ballot_sync(0xffffffffu, iseq);
            const bool sel = isgt || (iseq && (int)(eqrun + __popc(beq & lt)) < need);
            const uint32_t bsel = __ballot_sync(0xffffffffu, sel);
            if (sel) out[pos + __popc(bsel & lt)] = i;
            pos += __popc(bsel);
            eqrun += __popc(beq);
        }
    }
    __syncthreads();
}

// Same result as block_topk_sorted for T <= NT * R, with every score loaded ONCE: lane l of a warp keeps the keys of
// elements s0 + 32 j + l (j < R) of the warp's contiguous segment in registers, so the four histogram passes, the
// count and the ordered write-out run on registers only.
template <int NT, int R>
__device__ void block_topk_sorted_cached(const float* sc, int T, int k, int* out, uint32_t* sm) {
    constexpr int NW = NT / 32;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (k <= 0) return;
    if (k >= T) {
        for (int i = tid; i < T; i += NT) out[i] = i;
        return;
    }
    uint32_t* hist = sm;
    uint32_t* wcnt = sm + NW * 256;
    uint32_t* bc = wcnt + 4 * NW;

    int seg = (T + NW - 1) / NW;
    seg = (seg + 31) & ~31;  // <= 32 * R because T <= NT * R
    const int s0 = min(T, warp * seg), s1 = min(T, s0 + seg);
    uint32_t key[R];
    uint32_t have = 0;
#pragma unroll
    for (int j = 0; j < R; ++j) {
        const int i = s0 + j * 32 + lane;
        key[j] = 0u;
        if (i < s1) { key[j] = score_key(sc[i]); have |= 1u << j; }
    }

    uint32_t prefix = 0, mask = 0;
    int remaining = k;
#pragma unroll 1
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        for (int i = tid; i < NW * 256; i += NT) hist[i] = 0;
        __syncthreads();
        uint32_t* myh = hist + warp * 256;
#pragma unroll
        for (int j = 0; j < R; ++j) {
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
        for (int b = tid; b < 256; b += NT) {
            uint32_t t = 0;
#pragma unroll 4
            for (int w = 0; w < NW; ++w) t += hist[w * 256 + b];
            hist[b] = t;
        }
        __syncthreads();
        if (warp == 0) {
            uint32_t mine = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) mine += hist[255 - 8 * lane - j];
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
                    const uint32_t c = hist[d];
                    if (above + c >= (uint32_t)remaining) break;
                    above += c;
                }
                bc[0] = (uint32_t)d;
                bc[1] = (uint32_t)remaining - above;
            }
        }
        __syncthreads();
        prefix |= bc[0] << shift;
        mask |= 0xFFu << shift;
        remaining = (int)bc[1];
        __syncthreads();
    }
    const uint32_t thr = prefix;
    const int need = remaining;

    uint32_t gt = 0, eq = 0;
#pragma unroll
    for (int j = 0; j < R; ++j) {
        const bool in = (have >> j) & 1u;
        gt += __popc(__ballot_sync(0xffffffffu, in && key[j] > thr));
        eq += __popc(__ballot_sync(0xffffffffu, in && key[j] == thr));
    }
    if (lane == 0) { wcnt[warp] = gt; wcnt[NW + warp] = eq; }
    __syncthreads();
    if (warp == 0) {
        uint32_t eqp = 0, selp = 0;
        for (int base = 0; base < NW; base += 32) {
            const int w = base + lane;
            const uint32_t g = w < NW ? wcnt[w] : 0u, e = w < NW ? wcnt[NW + w] : 0u;
            uint32_t ei = e;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t v = __shfl_up_sync(0xffffffffu, ei, o);
                if (lane >= o) ei += v;
            }
            const uint32_t eex = eqp + ei - e;
            const uint32_t take = (uint32_t)max(0, min((int)e, need - (int)eex));
            const uint32_t sl = g + take;
            uint32_t si = sl;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t v = __shfl_up_sync(0xffffffffu, si, o);
                if (lane >= o) si += v;
            }
            if (w < NW) { wcnt[2 * NW + w] = selp + si - sl; wcnt[3 * NW + w] = eex; }
            eqp += __shfl_sync(0xffffffffu, ei, 31);
            selp += __shfl_sync(0xffffffffu, si, 31);
        }
    }
    __syncthreads();
    uint32_t pos = wcnt[2 * NW + warp], eqrun = wcnt[3 * NW + warp];
    const uint32_t lt = (1u << lane) - 1u;
#pragma unroll
    for (int j = 0; j < R; ++j) {
        const bool in = (have >> j) & 1u;
        const bool isgt = in && key[j] > thr, iseq = in && key[j] == thr;
        const uint32_t beq = __ballot_sync(0xffffffffu, iseq);
        const bool sel = isgt || (iseq && (int)(eqrun + __popc(beq & lt)) < need);
        const uint32_t bsel = __ballot_sync(0xffffffffu, sel);
        if (sel) out[pos + __popc(bsel & lt)] = s0 + j * 32 + lane;
        pos += __popc(bsel);
        eqrun += __popc(beq);
    }
    __syncthreads();
}

// Exact top-k for a SMALL k (k <= 32) over T <= NT * R scores: arg-max extraction instead of histogram passes.
// Every score becomes a 64-bit key (order-preserving score bits, then the complemented position, so that among equal
// scores the lower position is the larger key).  Each warp extracts the k best of its contiguous segment (lane i keeps
// the i-th best); a warp-wide maximum of a 64-bit key is two redux.sync instructions (upper words, then the lower
// words of the lanes that hold the winning upper word).  The NT/32 * k candidates meet in shared memory, where a
// candidate is kept when fewer than k candidates outrank it, and the kept positions are written in ascending order.
// Four barriers in all, against six per pass of the radix routine.  `cand` is NT 64-bit words of shared memory.
// All NT threads must call it.
__device__ __forceinline__ unsigned long long warp_max_u64(unsigned long long v) {
    const uint32_t hi = (uint32_t)(v >> 32), lo = (uint32_t)v;
    const uint32_t mh = __reduce_max_sync(0xffffffffu, hi);
    const uint32_t ml = __reduce_max_sync(0xffffffffu, hi == mh ? lo : 0u);
    return ((unsigned long long)mh << 32) | ml;
}

template <int R>
__device__ __forceinline__ unsigned long long warp_extract_topk(unsigned long long (&key)[R], int k, int lane) {
    unsigned long long mine = 0ull;
    for (int it = 0; it < k; ++it) {
        unsigned long long m = key[0];
#pragma unroll
        for (int j = 1; j < R; ++j) m = key[j] > m ? key[j] : m;
        m = warp_max_u64(m);
        if (lane == it) mine = m;
#pragma unroll
        for (int j = 0; j < R; ++j)
            if (key[j] == m) key[j] = 0ull;   // keys are unique (the position is part of them); 0 never wins again
    }
    return mine;
}

template <int NT, int R>
__device__ void block_topk_small(const float* sc, int T, int k, int* out, unsigned long long* cand) {
    constexpr int NW = NT / 32;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (k <= 0) return;
    unsigned long long key[R];
#pragma unroll
    for (int j = 0; j < R; ++j) {
        const int i = (warp * R + j) * 32 + lane;
        key[j] = i < T ? ((unsigned long long)score_key(sc[i]) << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)i) : 0ull;
    }
    const unsigned long long mine = warp_extract_topk<R>(key, k, lane);   // lane i < k holds this warp's i-th best
    if (lane < k) cand[warp * k + lane] = mine;                           // NW * k candidates, packed (0: no such score)
    __syncthreads();
    __shared__ int by_rank[32];  // position of the candidate that exactly r others outrank, r < k
    const int total = NW * k;    // <= NT because k <= 32
    if (tid < 32) by_rank[tid] = -1;
    __syncthreads();
    if (tid < total) {
        const unsigned long long me = cand[tid];
        if (me != 0ull) {
            int outranked = 0;
            for (int q = 0; q < total; ++q) outranked += cand[q] > me ? 1 : 0;
            if (outranked < k) by_rank[outranked] = (int)(0xFFFFFFFFu - (uint32_t)me);
        }
    }
    __syncthreads();
    if (tid < k) {   // ascending positions: a kept position goes to the slot numbered by how many kept ones lie below it
        const int pos = by_rank[tid];
        if (pos >= 0) {
            int lower = 0;
            for (int q = 0; q < k; ++q) lower += (by_rank[q] >= 0 && by_rank[q] < pos) ? 1 : 0;
            out[lower] = pos;
        }
    }
    __syncthreads();
}

// ---- Exact top-k without histogram passes, for k <= min(NT / 2, 256).
// The threads are cut into G >= 2k groups of consecutive lanes; the k-th largest of the G group maxima is a lower
// bound of the k-th largest score (the maxima are G distinct elements), and for scores in no particular order only
// about 0.7 G elements reach it.  Those survivors are appended to shared memory as 64-bit words (order-preserving
// score bits, then the complemented position, so that a greater word is a better rank and no two are equal); every
// survivor's rank is counted by a whole warp (lanes stride over the list, one ballot per 32 comparisons -- a single
// thread looping over the list pays a shared-memory latency per element), and the k best are written in ascending
// position the same way.  Six barriers, one atomic per warp; a row on which more than NT / 2 elements survive (long
// runs of equal scores, say) goes to the radix routine instead.  Same result as block_topk_sorted.  All NT threads
// must call these; `sm` is TopkSmem<NT>::WORDS words, 8-byte aligned:
//   gm = sm [NT]: group maxima, later the kept survivors' positions; surv = sm + NT [NT / 2 x 64 bit]; misc = sm + 3 NT.

// The pivot from every thread's maximum key m (0: the thread has no element).
template <int NT>
__device__ __forceinline__ uint32_t pivot_from_thread_maxima(uint32_t m, int k, uint32_t* sm) {
    static_assert(TopkSmem<NT>::WORDS >= 3 * NT + 4, "shared memory of the pivot routines");
    constexpr int NW = NT / 32;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    uint32_t* gm = sm;
    uint32_t* misc = sm + 3 * NT;
    int gs = 32;   // lanes per group: the largest power of two that leaves at least 2k groups
    while (gs > 1 && NT / gs < 2 * k) gs >>= 1;
    const int G = NT / gs;
    for (int o = 1; o < gs; o <<= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((tid & (gs - 1)) == 0) gm[tid / gs] = m;
    if (tid == 0) misc[1] = 0u;
    __syncthreads();
    for (int t = warp; t < G; t += NW) {   // the group maximum that exactly k - 1 others outrank is the pivot
        const uint32_t v = gm[t];
        int c = 0;
        for (int q0 = 0; q0 < G; q0 += 32) {
            const int q = q0 + lane;
            const uint32_t u = q < G ? gm[q] : 0u;
            c += __popc(__ballot_sync(0xffffffffu, q < G && (u > v || (u == v && q < t))));
        }
        if (c == k - 1 && lane == 0) misc[0] = v;
    }
    __syncthreads();
    return misc[0];
}

// First free slot for this lane's `cnt` survivors: a scan inside the warp, one atomic per warp.
template <int NT>
__device__ __forceinline__ uint32_t pivot_reserve_slots(uint32_t cnt, uint32_t* sm) {
    const int lane = threadIdx.x & 31;
    uint32_t incl = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    const uint32_t wtotal = __shfl_sync(0xffffffffu, incl, 31);
    uint32_t base = 0;
    if (lane == 0 && wtotal) base = atomicAdd(sm + 3 * NT + 1, wtotal);
    base = __shfl_sync(0xffffffffu, base, 0);
    return base + incl - cnt;
}

__device__ __forceinline__ unsigned long long pivot_word(uint32_t key, int pos) {
    return ((unsigned long long)key << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)pos);
}

// Ranks the `total` (<= NT / 2) survivors and writes the k best positions, ascending.  Ends with a barrier.
template <int NT>
__device__ __forceinline__ void pivot_rank_and_write(int total, int k, int* out, uint32_t* sm) {
    constexpr int NW = NT / 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t* gm = sm;
    const unsigned long long* surv = reinterpret_cast<const unsigned long long*>(sm + NT);
    for (int t = warp; t < total; t += NW) {   // gm[t]: the survivor's position if fewer than k others outrank it
        const unsigned long long mine = surv[t];
        int c = 0;
        for (int q0 = 0; q0 < total; q0 += 32) {
            const int q = q0 + lane;
            c += __popc(__ballot_sync(0xffffffffu, q < total && surv[min(q, total - 1)] > mine));
        }
        if (lane == 0) gm[t] = c < k ? 0xFFFFFFFFu - (uint32_t)mine : 0xFFFFFFFFu;
    }
    __syncthreads();
    for (int t = warp; t < total; t += NW) {
        const uint32_t mine = gm[t];
        if (mine == 0xFFFFFFFFu) continue;   // (warp-uniform)
        int pos = 0;
        for (int q0 = 0; q0 < total; q0 += 32) {
            const int q = q0 + lane;
            pos += __popc(__ballot_sync(0xffffffffu, q < total && gm[min(q, total - 1)] < mine));
        }
        if (lane == 0) out[pos] = (int)mine;
    }
    __syncthreads();
}

// Rows of up to NT * R scores: every score is loaded once and its key kept in a register.
template <int NT, int R>
__device__ void block_topk_pivot(const float* sc, int T, int k, int* out, uint32_t* sm) {
    constexpr int NW = NT / 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned long long* surv = reinterpret_cast<unsigned long long*>(sm + NT);
    int seg = (T + NW - 1) / NW;
    seg = (seg + 31) & ~31;  // <= 32 * R because T <= NT * R
    const int s0 = min(T, warp * seg), s1 = min(T, s0 + seg);
    uint32_t key[R];
    uint32_t m = 0;
    {
        float raw[R];   // (unconditional loads at clamped positions: all in flight together)
#pragma unroll
        for (int j = 0; j < R; ++j) raw[j] = sc[min(s0 + j * 32 + lane, T - 1)];
#pragma unroll
        for (int j = 0; j < R; ++j) {
            key[j] = s0 + j * 32 + lane < s1 ? score_key(raw[j]) : 0u;
            m = max(m, key[j]);
        }
    }
    const uint32_t pivot = pivot_from_thread_maxima<NT>(m, k, sm);
    uint32_t mask = 0;
#pragma unroll
    for (int j = 0; j < R; ++j)
        if (s0 + j * 32 + lane < s1 && key[j] >= pivot) mask |= 1u << j;
    uint32_t slot = pivot_reserve_slots<NT>(__popc(mask), sm);
#pragma unroll
    for (int j = 0; j < R; ++j) {
        if ((mask >> j) & 1u) {
            if (slot < (uint32_t)(NT / 2)) surv[slot] = pivot_word(key[j], s0 + j * 32 + lane);
            ++slot;
        }
    }
    __syncthreads();
    const int total = (int)sm[3 * NT + 1];
    if (total > NT / 2) {   // (the same decision in every thread)
        __syncthreads();
        block_topk_sorted_cached<NT, R>(sc, T, k, out, sm);
        return;
    }
    pivot_rank_and_write<NT>(total, k, out, sm);
}

// Rows of any length: three passes over the scores (thread maxima, survivor counts, survivor words), thread t taking
// the elements t, t + NT, ...; eight loads in flight per thread.
template <int NT>
__device__ void block_topk_pivot_stream(const float* sc, int T, int k, int* out, uint32_t* sm) {
    constexpr int U = 8;
    const int tid = threadIdx.x;
    unsigned long long* surv = reinterpret_cast<unsigned long long*>(sm + NT);
    uint32_t m = 0;
    for (int i0 = tid; i0 < T; i0 += U * NT) {
        float raw[U];
#pragma unroll
        for (int u = 0; u < U; ++u) raw[u] = sc[min(i0 + u * NT, T - 1)];
#pragma unroll
        for (int u = 0; u < U; ++u) m = max(m, i0 + u * NT < T ? score_key(raw[u]) : 0u);
    }
    const uint32_t pivot = pivot_from_thread_maxima<NT>(m, k, sm);
    uint32_t cnt = 0;
    for (int i0 = tid; i0 < T; i0 += U * NT) {
        float raw[U];
#pragma unroll
        for (int u = 0; u < U; ++u) raw[u] = sc[min(i0 + u * NT, T - 1)];
#pragma unroll
        for (int u = 0; u < U; ++u) cnt += (i0 + u * NT < T && score_key(raw[u]) >= pivot) ? 1u : 0u;
    }
    uint32_t slot = pivot_reserve_slots<NT>(cnt, sm);
    if (cnt) {
        for (int i0 = tid; i0 < T; i0 += U * NT) {
            float raw[U];
#pragma unroll
            for (int u = 0; u < U; ++u) raw[u] = sc[min(i0 + u * NT, T - 1)];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const uint32_t key = score_key(raw[u]);
                if (i0 + u * NT < T && key >= pivot) {
                    if (slot < (uint32_t)(NT / 2)) surv[slot] = pivot_word(key, i0 + u * NT);
                    ++slot;
                }
            }
        }
    }
    __syncthreads();
    const int total = (int)sm[3 * NT + 1];
    if (total > NT / 2) {   // (the same decision in every thread)
        __syncthreads();
        block_topk_sorted<NT>(sc, T, k, out, sm);
        return;
    }
    pivot_rank_and_write<NT>(total, k, out, sm);
}

#ifndef SKV_TOPK_PIVOT
#define SKV_TOPK_PIVOT 1   // 0: block_topk_fast never takes the pivot routine (for comparisons)
#endif

// Picks the register-cached routine when the row is short enough for R keys per thread.
template <int NT, int R>
__device__ __forceinline__ void block_topk_sorted_auto(const float* sc, int T, int k, int* out, uint32_t* sm) {
    if (T <= NT * R) block_topk_sorted_cached<NT, R>(sc, T, k, out, sm);
    else block_topk_sorted<NT>(sc, T, k, out, sm);
}

// The quickest exact routine for the problem: arg-max extraction for k <= 8 over rows of up to 16 scores per
// thread, the pivot routine for k up to min(NT / 2, 256) over rows of up to R scores per thread, the register-cached
// radix select for other rows of that length; longer rows: the streaming pivot routine for such k, the streaming radix
// select otherwise.  `sm` is TopkSmem<NT>::WORDS words (the small routine uses the first 2 * NT of them).  Output ascending.
template <int NT, int R>
__device__ __forceinline__ void block_topk_fast(const float* sc, int T, int k, int* out, uint32_t* sm) {
    static_assert(TopkSmem<NT>::WORDS >= 2 * NT, "candidate scratch of the small routine");
    unsigned long long* cand = reinterpret_cast<unsigned long long*>(sm);
    if (k >= T) {   // everything is kept
        for (int i = threadIdx.x; i < T; i += NT) out[i] = i;
        __syncthreads();
        return;
    }
    // The small routine's last round compares every candidate with every other ((NT/32 * k)^2 comparisons spread over
    // the CTA): it wins while that is a few hundred candidates and loses badly beyond (top-32 with 32 warps is 1024
    // candidates, a million comparisons: 25 us against 5 us for the radix passes).
    // The first round costs k extraction steps per warp: measured a loss already at k = 32 (token-sparse top-32 at 64K:
    // 134 us against 124 us with the radix passes), a gain at k = 8.
    const bool small = k <= 8 && (NT / 32) * k <= 256;
    if (small && T <= NT * 2) block_topk_small<NT, 2>(sc, T, k, out, cand);
    else if (small && T <= NT * 4) block_topk_small<NT, 4>(sc, T, k, out, cand);
    else if (small && T <= NT * 8) block_topk_small<NT, 8>(sc, T, k, out, cand);
    else if (small && T <= NT * 16) block_topk_small<NT, 16>(sc, T, k, out, cand);
    else if (SKV_TOPK_PIVOT && k > 0 && 2 * k <= NT && k <= 256 && T <= NT * R) block_topk_pivot<NT, R>(sc, T, k, out, sm);
    else if (SKV_TOPK_PIVOT && k > 0 && 2 * k <= NT && k <= 256) block_topk_pivot_stream<NT>(sc, T, k, out, sm);
    else block_topk_sorted_auto<NT, R>(sc, T, k, out, sm);
}

}  // namespace skv
