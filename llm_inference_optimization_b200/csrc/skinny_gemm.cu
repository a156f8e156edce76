// Skinny GEMM of the decode step: out[M, N] = x[M, K] . w[K, N] with M <= 16 rows (the batch of one decode step),
// 16-bit inputs, fp32 accumulation.
//
// The reference runs these projections as Hugging Face nn.Linear modules (the model it patches,
// benchmarks/llama_integration_benchmark.py:266-279), i.e. library GEMMs; with 16 rows they are pure weight
// streaming (2 FLOP per weight byte).  This kernel is built like the decode-attention kernels:
//   * a column tile is 256 columns wide, so every row of w contributes 512 contiguous bytes to a stage (narrow
//     tiles turn the stream into scattered 128-byte DRAM accesses and cost a third of the bandwidth);
//   * "stream-K": the (column tile, 32-row block) space of w is flattened and cut into one contiguous range per
//     CTA of a grid of exactly two CTAs per SM, so every CTA streams the same number of bytes whatever N and K are;
//     a range may cross from one column tile into the next (the accumulators are flushed there);
//   * a producer lane issues TMA boxes (four of 32 rows x 64 columns of w, 128-byte swizzle, evict-first; the
//     matching 16 x 32 slice of x, 64-byte swizzle, evict-last) into a 6-stage mbarrier ring; four consumer warps
//     take 64 columns each: ldmatrix (transposed for w) + mma.sync.m16n8k16 with the 16 rows of x as the M side;
//   * a column tile that several CTAs contributed to is finished by the last of them (fp32 partials in the
//     workspace, an atomic ticket per tile; no spin wait, no second launch).
// Columns past N (N need only be a multiple of 64) are zero-filled by the TMA unit and never stored.
// Every wait is bounded; a wait that runs out sets SKV_DEV_TIMEOUT in the status word at offset 0 of the workspace.
#include <cuda_bf16.h>

#include "skv_common.cuh"
#include "skv_tmap.cuh"

namespace skv {
namespace sgemm {

constexpr int BN = 256;                      // columns per tile
constexpr int BK = 32;                       // rows of w per pipeline stage
constexpr int BOX_BYTES = BK * 128;          // one [32][64] box of w
constexpr int W_BYTES = 4 * BOX_BYTES;       // 16 KB
constexpr int X_BYTES = 16 * BK * 2;         // 1 KB: [16][32], 64-byte rows
constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
constexpr int STAGES = 6;
constexpr int CONSUMERS = 4;
constexpr int THREADS = (CONSUMERS + 1) * 32;
constexpr size_t HEAD_BYTES = 65536;         // status word + one ticket per column tile
constexpr int MAX_N = 256 * 16320;
constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 2 * STAGES * 8 + 16 + 1024;

struct Params {
    void* out;            // [M, N] 16-bit, row-major
    float* partial;       // [n_tiles, max_contrib, 16, BN]
    int* tickets;         // [n_tiles], zero between launches
    int* status;
    int M, N, KB, n_tiles, max_contrib;
    long long total, per;  // blocks in all, blocks per CTA
};

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    if (BF16) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<const uint32_t*>(&v);
    }
    return pack_half2(a, b);
}

template <bool BF16>
__global__ void __launch_bounds__(THREADS, 2)
skinny_gemm_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t ring = smem_u32(smem);
    const uint32_t full_bar = ring + STAGES * STAGE_BYTES, empty_bar = full_bar + STAGES * 8;
    int* last_flag = reinterpret_cast<int*>(smem + STAGES * STAGE_BYTES + 2 * STAGES * 8);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long g0 = min(p.total, (long long)blockIdx.x * p.per), g1 = min(p.total, g0 + p.per);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar + s * 8, 1);
            mbar_init(empty_bar + s * 8, CONSUMERS);
        }
        fence_barrier_init();
    }
    __syncthreads();

    if (warp == CONSUMERS) {   // producer: one lane, five boxes per stage
        if (lane == 0) {
            tma_prefetch_desc(&tmW);
            tma_prefetch_desc(&tmX);
            const uint64_t stream_once = l2_policy_evict_first(), keep = l2_policy_evict_last();
            int s = 0;
            uint32_t ph = 0;
            long long it = 0;
            int tile = (int)(g0 / p.KB), kb = (int)(g0 - (long long)tile * p.KB);
            for (long long gi = g0; gi < g1; ++gi, ++it) {
                if (it >= STAGES && !mbar_wait(empty_bar + s * 8, ph ^ 1u)) {
                    atomicOr(p.status, SKV_DEV_TIMEOUT);
                    break;
                }
                const uint32_t dst = ring + s * STAGE_BYTES, bar = full_bar + s * 8;
                mbar_expect_tx(bar, STAGE_BYTES);
#pragma unroll
                for (int bx = 0; bx < 4; ++bx)
                    tma_load_2d(dst + bx * BOX_BYTES, &tmW, bar, tile * BN + bx * 64, kb * BK, stream_once);
                tma_load_2d(dst + W_BYTES, &tmX, bar, kb * BK, 0, keep);
                if (++s == STAGES) { s = 0; ph ^= 1u; }
                if (++kb == p.KB) { kb = 0; ++tile; }
            }
        }
        return;
    }

    // consumers: warp w owns columns 64w .. 64w+63 of the tile, i.e. box w of every stage
    const int g = lane >> 2, tq = lane & 3;
    const int m = lane >> 3, r8 = lane & 7;
    const int a_row = (m & 1) * 8 + r8;           // x row this lane addresses for ldmatrix
    int s = 0;
    uint32_t ph = 0;
    long long gpos = g0;
    while (gpos < g1) {
        const int tile = (int)(gpos / p.KB);
        const int kb0 = (int)(gpos - (long long)tile * p.KB);
        const int nblk = (int)min((long long)(p.KB - kb0), g1 - gpos);
        float acc[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
        for (int i = 0; i < nblk; ++i) {
            int ok = 1;
            if (lane == 0) ok = mbar_wait(full_bar + s * 8, ph) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) {
                if (lane == 0) atomicOr(p.status, SKV_DEV_TIMEOUT);
                return;
            }
            const uint32_t wbase = ring + s * STAGE_BYTES + warp * BOX_BYTES, xbase = ring + s * STAGE_BYTES + W_BYTES;
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk) {
                uint32_t a[4];
                const int kchunk = kk * 2 + (m >> 1);            // 16-byte chunk of the 64-byte x row (64-byte swizzle)
                ldsm_x4(xbase + a_row * 64 + ((kchunk ^ ((a_row >> 1) & 3)) << 4), a[0], a[1], a[2], a[3]);
                const int krow = kk * 16 + (m & 1) * 8 + r8;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4_t(wbase + krow * 128 + (((2 * j + (m >> 1)) ^ (krow & 7)) << 4), b0, b1, b2, b3);
                    if (BF16) {
                        mma_bf16(acc[2 * j], a, b0, b1);
                        mma_bf16(acc[2 * j + 1], a, b2, b3);
                    } else {
                        mma_f16(acc[2 * j], a, b0, b1);
                        mma_f16(acc[2 * j + 1], a, b2, b3);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar + s * 8);
            if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        gpos += nblk;

        // ---- this CTA's share of the tile is summed: write it out, or hand it to the tile's last contributor
        const long long tfirst = (long long)tile * p.KB;
        const int c_first = (int)(tfirst / p.per), c_last = (int)((tfirst + p.KB - 1) / p.per);
        const int count = c_last - c_first + 1, ord = (int)blockIdx.x - c_first;
        const int col = warp * 64 + tq * 2;      // + 8 j
        uint16_t* out = static_cast<uint16_t*>(p.out);
        if (count == 1) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const long long c = (long long)tile * BN + col + j * 8;
                if (c >= p.N) continue;
                if (g < p.M) *reinterpret_cast<uint32_t*>(out + (long long)g * p.N + c) = pack2<BF16>(acc[j][0], acc[j][1]);
                if (g + 8 < p.M) *reinterpret_cast<uint32_t*>(out + (long long)(g + 8) * p.N + c) = pack2<BF16>(acc[j][2], acc[j][3]);
            }
            continue;
        }
        float* mine = p.partial + ((long long)tile * p.max_contrib + ord) * (16 * BN);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            *reinterpret_cast<float2*>(mine + g * BN + col + j * 8) = make_float2(acc[j][0], acc[j][1]);
            *reinterpret_cast<float2*>(mine + (g + 8) * BN + col + j * 8) = make_float2(acc[j][2], acc[j][3]);
        }
        __threadfence();
        named_bar_sync(1, CONSUMERS * 32);
        if (threadIdx.x == 0) {
            const int ticket = atomicAdd(&p.tickets[tile], 1);
            const int last = ticket == count - 1;
            if (last) p.tickets[tile] = 0;   // ready for the next launch on this workspace
            *last_flag = last;
        }
        named_bar_sync(1, CONSUMERS * 32);
        const bool last = *last_flag != 0;
        named_bar_sync(1, CONSUMERS * 32);   // everybody has read the flag before the next tile may rewrite it
        if (!last) continue;
        __threadfence();
        const float* base = p.partial + (long long)tile * p.max_contrib * (16 * BN) + g * BN + col;
        float2 lo[8], hi[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) lo[j] = hi[j] = make_float2(0.f, 0.f);
#pragma unroll 2
        for (int o = 0; o < count; ++o) {   // contributions in CTA order: the sum does not depend on who finished last
            float2 u[8], v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                u[j] = __ldcg(reinterpret_cast<const float2*>(base + o * (16 * BN) + j * 8));
                v[j] = __ldcg(reinterpret_cast<const float2*>(base + o * (16 * BN) + 8 * BN + j * 8));
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                lo[j].x += u[j].x; lo[j].y += u[j].y;
                hi[j].x += v[j].x; hi[j].y += v[j].y;
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const long long c = (long long)tile * BN + col + j * 8;
            if (c >= p.N) continue;
            if (g < p.M) *reinterpret_cast<uint32_t*>(out + (long long)g * p.N + c) = pack2<BF16>(lo[j].x, lo[j].y);
            if (g + 8 < p.M) *reinterpret_cast<uint32_t*>(out + (long long)(g + 8) * p.N + c) = pack2<BF16>(hi[j].x, hi[j].y);
        }
    }
}

struct Plan {
    int n_tiles, KB, ctas, max_contrib;
    long long total, per;
    size_t off_tickets, off_partial, bytes;
};

// Fewest 16 KB blocks of w a CTA should stream when the problem is too small to give every CTA that many: below it a
// CTA is all start-up, and every extra contributor to a column tile lengthens the tile's final sum.
inline int& min_blocks() {
    static int v = 16;
    return v;
}

inline Plan make_plan(int K, int N, int device) {
    Plan pl;
    pl.n_tiles = (N + BN - 1) / BN;
    pl.KB = K / BK;
    pl.total = (long long)pl.n_tiles * pl.KB;
    const long long max_ctas = (long long)sm_count(device) * 2;
    const long long even = (pl.total + max_ctas - 1) / max_ctas;
    const int floor_blocks = min_blocks();
    if (even >= floor_blocks) {
        pl.per = even;                               // large problem: equal ranges, cut wherever they fall
    } else if (pl.KB <= floor_blocks) {
        pl.per = pl.KB;                              // one CTA per (short) column tile, no partial sums
    } else {
        const int shares = pl.KB / floor_blocks;     // a few equal shares of every column tile
        pl.per = (pl.KB + shares - 1) / shares;
    }
    pl.ctas = (int)((pl.total + pl.per - 1) / pl.per);
    pl.max_contrib = (int)((pl.KB + pl.per - 1) / pl.per) + 1;
    // status word and tickets in a head region of fixed size: a later, wider problem must not find an earlier one's
    // partial sums where its tickets live (N <= 256 * 16320 columns)
    pl.off_tickets = 256;
    pl.off_partial = HEAD_BYTES;
    pl.bytes = pl.off_partial + (size_t)pl.n_tiles * pl.max_contrib * 16 * BN * sizeof(float);
    return pl;
}

}  // namespace sgemm
}  // namespace skv

using namespace skv;

extern "C" {

// Tuning knob for experiments: the fewest 16 KB blocks of w per CTA on small problems (1..64).
int skv_skinny_gemm_set_min_blocks(int blocks) {
    if (blocks < 1 || blocks > 64) return fail(SKV_ERR_BAD_ARG, "min blocks %d out of range 1..64", blocks);
    sgemm::min_blocks() = blocks;
    return SKV_OK;
}

// Workspace of skv_skinny_gemm (0 when the shape is not supported): zero-filled once before its first use.
size_t skv_skinny_gemm_workspace_bytes(int M, int K, int N, int device) {
    if (M <= 0 || M > 16 || K <= 0 || N <= 0 || K % sgemm::BK || N % 64 || N > sgemm::MAX_N) return 0;
    return sgemm::make_plan(K, N, device).bytes;
}

int skv_skinny_gemm(const void* x, const void* w, void* out, void* workspace, size_t workspace_bytes, int M, int K, int N,
                    int is_bf16, int device, void* stream) {
    if (!x || !w || !out) return fail(SKV_ERR_BAD_ARG, "skv_skinny_gemm: null tensor pointer");
    if (M <= 0 || M > 16) return fail(SKV_ERR_UNSUPPORTED, "skv_skinny_gemm serves 1..16 rows, got %d", M);
    if (K <= 0 || N <= 0 || K % sgemm::BK || N % 64)
        return fail(SKV_ERR_UNSUPPORTED, "K must be a multiple of %d and N of 64 (K=%d, N=%d)", sgemm::BK, K, N);
    if (N > sgemm::MAX_N) return fail(SKV_ERR_UNSUPPORTED, "N=%d exceeds %d columns", N, sgemm::MAX_N);
    if ((reinterpret_cast<uintptr_t>(out) & 3)) return fail(SKV_ERR_BAD_ARG, "out must be 4-byte aligned");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(SKV_ERR_CUDA, "cannot switch to device %d", device);
    const sgemm::Plan pl = sgemm::make_plan(K, N, device);
    if (!workspace || workspace_bytes < pl.bytes)
        return fail(SKV_ERR_WORKSPACE, "workspace of %zu bytes is smaller than the %zu required", workspace_bytes, pl.bytes);
    if (reinterpret_cast<uintptr_t>(workspace) & 255) return fail(SKV_ERR_WORKSPACE, "workspace must be 256-byte aligned");

    CUtensorMap tmW, tmX;
    int rc = make_matrix_tmap(&tmW, w, K, N, N, sgemm::BK, 64, is_bf16 != 0);
    if (rc) return rc;
    rc = make_matrix_tmap(&tmX, x, M, K, K, 16, sgemm::BK, is_bf16 != 0);
    if (rc) return rc;

    sgemm::Params p;
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    p.out = out;
    p.status = reinterpret_cast<int*>(ws);
    p.tickets = reinterpret_cast<int*>(ws + pl.off_tickets);
    p.partial = reinterpret_cast<float*>(ws + pl.off_partial);
    p.M = M; p.N = N; p.KB = pl.KB; p.n_tiles = pl.n_tiles; p.max_contrib = pl.max_contrib;
    p.total = pl.total; p.per = pl.per;

    static bool configured[64] = {false};
    if (device < 64 && !configured[device]) {
        SKV_CUDA_TRY(cudaFuncSetAttribute(sgemm::skinny_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sgemm::SMEM));
        SKV_CUDA_TRY(cudaFuncSetAttribute(sgemm::skinny_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sgemm::SMEM));
        configured[device] = true;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (is_bf16) sgemm::skinny_gemm_kernel<true><<<pl.ctas, sgemm::THREADS, sgemm::SMEM, st>>>(tmW, tmX, p);
    else sgemm::skinny_gemm_kernel<false><<<pl.ctas, sgemm::THREADS, sgemm::SMEM, st>>>(tmW, tmX, p);
    SKV_CUDA_TRY(cudaGetLastError());
    return SKV_OK;
}

}  // extern "C"
