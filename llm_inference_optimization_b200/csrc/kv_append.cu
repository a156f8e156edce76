// Decode-step glue in front of the attention kernel: rotary embedding of the new token's query and key,
// quantisation of its key and value rows (FP8-E4M3 or INT8, one fp32 scale per row) and their store into the
// paged cache at position seq_lens[b] -- one launch instead of the concatenate-and-copy the reference does
// (DynamicCache.update plus permute().contiguous() of the whole cache per layer and token,
// benchmarks/llama_integration_benchmark.py:173,302-303; benchmarks/profile_fused_gqa.py:143-144).
//
// qkv : [B, (Hq + 2 Hkv) * D] bf16 or fp16, the output of the fused q/k/v projection (q heads, then k, then v)
// q_out : [B, Hq, D] fp16, rotated query for the decode kernel
// pools : as for skv_gqa_decode_paged (separate or fused page records; addressed through strides); with SKV_V_INT4
//         the value row is quantised to 4 bits (scale = amax / 7) and packed two channels per byte
// One warp per (b, head): D = 128 -> 4 channels per lane; rotate-half pairs channel d with d + D/2.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "skv_common.cuh"

namespace skv {
namespace app {

constexpr int D = 128;
constexpr int THREADS = 128;

struct Params {
    const void* qkv;
    __half* q_out;
    uint8_t* k_codes; uint8_t* v_codes;   // element (page,h,slot,d) at page*sp + h*sh + slot*ss + d
    float* k_scale; float* v_scale;       // element (page,h,slot) at page*csp + h*csh + slot
    const int* page_table;                // [B, max_pages] or null
    const int* seq_lens;                  // [B]: position the new token takes
    long long sp, sh, ss, csp, csh;
    int B, Hq, Hkv, page_size, max_pages, num_pages, kv_dtype;
    int v4;                               // V rows are stored as 4-bit codes, 64 bytes per token (mixed-precision pages)
    int* status;                          // optional device status word (SKV_DEV_BAD_PAGE)
    float log2_theta;
    __half* meta;                         // optional [B, Hkv, nb, 2, D] min/max block metadata to keep current
    int meta_block, meta_nb;
};

template <typename T>
__device__ __forceinline__ float load_elem(const void* p, long long i);
template <>
__device__ __forceinline__ float load_elem<__half>(const void* p, long long i) {
    return __half2float(static_cast<const __half*>(p)[i]);
}
template <>
__device__ __forceinline__ float load_elem<__nv_bfloat16>(const void* p, long long i) {
    return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}

// grid: ceil(B * (Hq + 2 Hkv) / 4) CTAs of 4 warps
template <typename T>
__global__ void __launch_bounds__(THREADS)
rope_quant_append_kernel(const Params p) {
    // A decode kernel launched behind this one as a programmatic dependent (SKV_EARLY_EXCEPT_LAST) may start now: it
    // streams everything but the tile of the token stored here, and waits for this grid before it touches that
    // tile or the rotated query.
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads = p.Hq + 2 * p.Hkv;
    const long long item = (long long)blockIdx.x * (THREADS / 32) + warp;
    if (item >= (long long)p.B * heads) return;
    const int b = (int)(item / heads), hh = (int)(item % heads);
    const int pos = p.seq_lens[b];
    const long long src = ((long long)b * heads + hh) * D;
    // lane holds channels lane*2, lane*2+1 of the first half and the same of the second half
    float lo0 = load_elem<T>(p.qkv, src + lane * 2), lo1 = load_elem<T>(p.qkv, src + lane * 2 + 1);
    float hi0 = load_elem<T>(p.qkv, src + D / 2 + lane * 2), hi1 = load_elem<T>(p.qkv, src + D / 2 + lane * 2 + 1);
    const bool is_v = hh >= p.Hq + p.Hkv;
    if (!is_v) {  // rotate-half RoPE: (x_d, x_{d+D/2}) -> (x_d cos - x_{d+D/2} sin, x_{d+D/2} cos + x_d sin)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int d = lane * 2 + j;
            const float inv_freq = exp2f(-p.log2_theta * (float)(2 * d) / (float)D);
            float sn, cs;
            sincosf((float)pos * inv_freq, &sn, &cs);
            float& a = j ? lo1 : lo0;
            float& c = j ? hi1 : hi0;
            const float ra = a * cs - c * sn, rc = c * cs + a * sn;
            a = ra;
            c = rc;
        }
    }
    if (hh < p.Hq) {
        __half* dst = p.q_out + ((long long)b * p.Hq + hh) * D;
        *reinterpret_cast<__half2*>(dst + lane * 2) = __floats2half2_rn(lo0, lo1);
        *reinterpret_cast<__half2*>(dst + D / 2 + lane * 2) = __floats2half2_rn(hi0, hi1);
        return;
    }
    // key or value row: per-row scale = amax / qmax, round-to-nearest-even codes
    const int h = is_v ? hh - p.Hq - p.Hkv : hh - p.Hq;
    float amax = fmaxf(fmaxf(fabsf(lo0), fabsf(lo1)), fmaxf(fabsf(hi0), fabsf(hi1)));
    amax = warp_max(amax);
    const bool v4 = is_v && p.v4;
    const float qmax = v4 ? 7.f : p.kv_dtype == SKV_KV_E4M3 ? 448.f : 127.f;
    const float scale = amax > 0.f ? __fdiv_rn(amax, qmax) : 1.f;
    const float x[4] = {lo0, lo1, hi0, hi1};
    uint32_t code[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float y = __fdiv_rn(x[i], scale);
        if (v4)
            code[i] = (uint32_t)(max(-7, min(7, __float2int_rn(y))) + 8);
        else if (p.kv_dtype == SKV_KV_E4M3)
            code[i] = (uint32_t)__nv_cvt_float_to_fp8(fminf(fmaxf(y, -448.f), 448.f), __NV_SATFINITE, __NV_E4M3);
        else
            code[i] = (uint32_t)max(-127, min(127, __float2int_rn(y))) & 0xFFu;
    }
    const int lp = pos / p.page_size, slot = pos - lp * p.page_size;
    if (pos < 0 || lp >= p.max_pages) return;   // no room left in this sequence's page list: nothing is stored
    const int page = p.page_table ? p.page_table[(long long)b * p.max_pages + lp] : b * p.max_pages + lp;
    if ((unsigned)page >= (unsigned)p.num_pages) {   // a stale or corrupt table entry: store nothing, report it
        if (lane == 0 && p.status) atomicOr(p.status, SKV_DEV_BAD_PAGE);
        return;
    }
    if (v4) {   // byte j of the 64-byte row: channel 2j in the low nibble, 2j+1 in the high one
        uint8_t* row = p.v_codes + SKV_INDEX(page, p.num_pages) * p.sp + h * p.sh + SKV_INDEX(slot, p.page_size) * (D / 2);
        row[lane] = (uint8_t)(code[0] | (code[1] << 4));
        row[D / 4 + lane] = (uint8_t)(code[2] | (code[3] << 4));
    } else {
        uint8_t* row = (is_v ? p.v_codes : p.k_codes) + SKV_INDEX(page, p.num_pages) * p.sp + h * p.sh + SKV_INDEX(slot, p.page_size) * p.ss;
        *reinterpret_cast<uint16_t*>(row + lane * 2) = (uint16_t)(code[0] | (code[1] << 8));
        *reinterpret_cast<uint16_t*>(row + D / 2 + lane * 2) = (uint16_t)(code[2] | (code[3] << 8));
    }
    if (lane == 0) (is_v ? p.v_scale : p.k_scale)[page * p.csp + h * p.csh + slot] = scale;

    // Keep the Quest metadata of the key's block current: min/max with the DEQUANTISED new key (code * scale),
    // starting afresh when the token opens a new block.  One warp owns a (b, head) row, so no other writer exists.
    if (!is_v && p.meta) {
        const int blk = pos / p.meta_block;
        if (blk < p.meta_nb) {
            const bool fresh = pos - blk * p.meta_block == 0;
            __half* mn = p.meta + ((((long long)b * p.Hkv + h) * p.meta_nb + blk) * 2) * D;
            __half* mx = mn + D;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int d = (i < 2 ? 0 : D / 2) + lane * 2 + (i & 1);
                float v;
                if (p.kv_dtype == SKV_KV_E4M3) {
                    const __half_raw hr = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)code[i], __NV_E4M3);
                    v = __half2float(*reinterpret_cast<const __half*>(&hr)) * scale;
                } else {
                    v = (float)(int)(int8_t)code[i] * scale;
                }
                const float lo = fresh ? v : fminf(__half2float(mn[d]), v);
                const float hi = fresh ? v : fmaxf(__half2float(mx[d]), v);
                mn[d] = __float2half_rn(lo);
                mx[d] = __float2half_rn(hi);
            }
        }
    }
}

}  // namespace app
}  // namespace skv

using namespace skv;

extern "C" {

int skv_rope_quant_append(const void* qkv, int qkv_is_bf16, void* q_out, void* k_pool, void* v_pool, float* k_scale_pool,
                          float* v_scale_pool, const int* page_table, const int* seq_lens, int B, int Hq, int Hkv,
                          int D, int kv_dtype, int page_size, int max_pages, long long pool_stride_page,
                          long long pool_stride_head, long long pool_stride_slot, long long scale_stride_page,
                          long long scale_stride_head, float rope_theta, void* meta, int meta_block_size,
                          int meta_num_blocks, int num_pages, int* status, int device, void* stream) {
    if (!qkv || !q_out || !k_pool || !v_pool || !k_scale_pool || !v_scale_pool || !seq_lens)
        return fail(SKV_ERR_BAD_ARG, "skv_rope_quant_append: null pointer");
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || page_size <= 0 || max_pages <= 0 || num_pages <= 0)
        return fail(SKV_ERR_BAD_ARG, "skv_rope_quant_append: sizes must be positive");
    if (D != app::D) return fail(SKV_ERR_UNSUPPORTED, "head dim %d not supported (128)", D);
    const int v4 = (kv_dtype & SKV_V_INT4) ? 1 : 0;   // V rows as 4-bit codes, 64 bytes per token slot
    kv_dtype &= ~SKV_V_INT4;
    if (kv_dtype != SKV_KV_I8 && kv_dtype != SKV_KV_E4M3) return fail(SKV_ERR_UNSUPPORTED, "kv_dtype %d is not an 8-bit type", kv_dtype);
    if (!(rope_theta > 1.f)) return fail(SKV_ERR_BAD_ARG, "rope_theta must exceed 1");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(SKV_ERR_CUDA, "cannot switch to device %d", device);
    app::Params p;
    p.qkv = qkv; p.q_out = static_cast<__half*>(q_out);
    p.k_codes = static_cast<uint8_t*>(k_pool); p.v_codes = static_cast<uint8_t*>(v_pool);
    p.k_scale = k_scale_pool; p.v_scale = v_scale_pool;
    p.page_table = page_table; p.seq_lens = seq_lens;
    p.sp = pool_stride_page; p.sh = pool_stride_head; p.ss = pool_stride_slot;
    p.csp = scale_stride_page; p.csh = scale_stride_head;
    p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.page_size = page_size; p.max_pages = max_pages; p.kv_dtype = kv_dtype;
    p.num_pages = num_pages; p.status = status;
    p.v4 = v4;
    p.log2_theta = log2f(rope_theta);
    p.meta = static_cast<__half*>(meta);
    p.meta_block = meta_block_size > 0 ? meta_block_size : 1;
    p.meta_nb = meta ? meta_num_blocks : 0;
    const long long items = (long long)B * (Hq + 2 * Hkv);
    const unsigned blocks = (unsigned)((items + 3) / 4);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (qkv_is_bf16) app::rope_quant_append_kernel<__nv_bfloat16><<<blocks, app::THREADS, 0, st>>>(p);
    else app::rope_quant_append_kernel<__half><<<blocks, app::THREADS, 0, st>>>(p);
    SKV_CUDA_TRY(cudaGetLastError());
    return SKV_OK;
}

}  // extern "C"

SKV_BOUNDS_GETTER(skv_debug_bounds_kv_append)
