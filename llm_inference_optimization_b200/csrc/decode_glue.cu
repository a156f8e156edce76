// Small fused kernels of the decode step around the attention call: residual add + RMSNorm, and SiLU(gate) * up.
// With 16 rows per step these ops are launch- and latency-bound; as separate framework kernels (add, norm,
// slice, silu, mul) they cost about 30 us per layer, a sixth of an 8-way tensor-parallel step.
//
// The reference runs the Hugging Face Llama modules for this part (LlamaRMSNorm / LlamaMLP inside the model it
// patches, benchmarks/llama_integration_benchmark.py:266-279); the sum and the activation are rounded to the
// storage type where the separate framework ops would round them.
#include <cuda_bf16.h>

#include "skv_common.cuh"

namespace skv {
namespace glue {

constexpr int NORM_THREADS = 256;

template <typename T> struct Elem;
template <> struct Elem<__half> {
    static __device__ __forceinline__ float to_f(uint16_t b) { return __half2float(__ushort_as_half(b)); }
    static __device__ __forceinline__ uint16_t from_f(float x) { return __half_as_ushort(__float2half_rn(x)); }
};
template <> struct Elem<__nv_bfloat16> {
    static __device__ __forceinline__ float to_f(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }
    static __device__ __forceinline__ uint16_t from_f(float x) { return __bfloat16_as_ushort(__float2bfloat16_rn(x)); }
};

template <typename T>
__device__ __forceinline__ void unpack8h(const uint4& v, float (&x)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        x[2 * i] = Elem<T>::to_f((uint16_t)(w[i] & 0xFFFFu));
        x[2 * i + 1] = Elem<T>::to_f((uint16_t)(w[i] >> 16));
    }
}

template <typename T>
__device__ __forceinline__ uint4 pack8h(const float (&x)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = (uint32_t)Elem<T>::from_f(x[2 * i]) | ((uint32_t)Elem<T>::from_f(x[2 * i + 1]) << 16);
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// One CTA per row.  resid <- round(resid + delta) (delta optional); out <- round(resid * rsqrt(mean(resid^2) + eps) * weight),
// fp32 throughout with one rounding at the end (torch.nn.functional.rms_norm's arithmetic).
// hidden <= NORM_THREADS * 8 * MAXV elements, a multiple of 8.
template <typename T, int MAXV>
__global__ void __launch_bounds__(NORM_THREADS)
residual_rmsnorm_kernel(const uint16_t* __restrict__ delta, uint16_t* __restrict__ resid, const uint16_t* __restrict__ weight,
                        uint16_t* __restrict__ out, int hidden, float eps) {
    __shared__ float red[NORM_THREADS / 32];
    __shared__ float bcast;
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long long base = (long long)row * hidden;
    float x[MAXV][8];
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
        const int c = (v * NORM_THREADS + tid) * 8;
        if (c < hidden) {
            unpack8h<T>(*reinterpret_cast<const uint4*>(resid + base + c), x[v]);
            if (delta) {
                float d[8];
                unpack8h<T>(*reinterpret_cast<const uint4*>(delta + base + c), d);
#pragma unroll
                for (int i = 0; i < 8; ++i) x[v][i] = Elem<T>::to_f(Elem<T>::from_f(x[v][i] + d[i]));
                *reinterpret_cast<uint4*>(resid + base + c) = pack8h<T>(x[v]);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) ss = fmaf(x[v][i], x[v][i], ss);
        }
    }
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    if (warp == 0) {
        float t = lane < NORM_THREADS / 32 ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) bcast = rsqrtf(t / (float)hidden + eps);
    }
    __syncthreads();
    const float inv = bcast;
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
        const int c = (v * NORM_THREADS + tid) * 8;
        if (c < hidden) {
            float w[8], y[8];
            unpack8h<T>(*reinterpret_cast<const uint4*>(weight + c), w);
#pragma unroll
            for (int i = 0; i < 8; ++i) y[i] = x[v][i] * inv * w[i];
            *reinterpret_cast<uint4*>(out + base + c) = pack8h<T>(y);
        }
    }
}

// out[r, c] = round(round(silu(gate[r, c])) * up[r, c]) with gate = gate_up[r, c], up = gate_up[r, inter + c]
template <typename T>
__global__ void __launch_bounds__(256)
silu_mul_kernel(const uint16_t* __restrict__ gate_up, uint16_t* __restrict__ out, int rows, int inter) {
    const long long per_row = inter / 8;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * per_row) return;
    const long long r = i / per_row, c = (i - r * per_row) * 8;
    float g[8], u[8], y[8];
    unpack8h<T>(*reinterpret_cast<const uint4*>(gate_up + r * 2 * inter + c), g);
    unpack8h<T>(*reinterpret_cast<const uint4*>(gate_up + r * 2 * inter + inter + c), u);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const float s = g[k] / (1.f + __expf(-g[k]));
        y[k] = Elem<T>::to_f(Elem<T>::from_f(s)) * u[k];
    }
    *reinterpret_cast<uint4*>(out + r * inter + c) = pack8h<T>(y);
}

}  // namespace glue
}  // namespace skv

using namespace skv;

extern "C" {

int skv_residual_rmsnorm(const void* delta, void* resid, const void* weight, void* out, int rows, int hidden, float eps,
                         int is_bf16, int device, void* stream) {
    if (!resid || !weight || !out) return fail(SKV_ERR_BAD_ARG, "skv_residual_rmsnorm: null pointer");
    if (rows <= 0 || hidden <= 0 || hidden % 8) return fail(SKV_ERR_BAD_ARG, "rows must be positive and hidden a positive multiple of 8");
    if (hidden > glue::NORM_THREADS * 8 * 4) return fail(SKV_ERR_UNSUPPORTED, "hidden %d exceeds %d", hidden, glue::NORM_THREADS * 8 * 4);
    if ((reinterpret_cast<uintptr_t>(resid) | reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(out) |
         reinterpret_cast<uintptr_t>(delta)) & 15)
        return fail(SKV_ERR_BAD_ARG, "skv_residual_rmsnorm: tensors must be 16-byte aligned");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(SKV_ERR_CUDA, "cannot switch to device %d", device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    auto* d = static_cast<const uint16_t*>(delta);
    auto* r = static_cast<uint16_t*>(resid);
    auto* w = static_cast<const uint16_t*>(weight);
    auto* o = static_cast<uint16_t*>(out);
    const bool small = hidden <= glue::NORM_THREADS * 8 * 2;
    if (is_bf16) {
        if (small) glue::residual_rmsnorm_kernel<__nv_bfloat16, 2><<<rows, glue::NORM_THREADS, 0, st>>>(d, r, w, o, hidden, eps);
        else glue::residual_rmsnorm_kernel<__nv_bfloat16, 4><<<rows, glue::NORM_THREADS, 0, st>>>(d, r, w, o, hidden, eps);
    } else {
        if (small) glue::residual_rmsnorm_kernel<__half, 2><<<rows, glue::NORM_THREADS, 0, st>>>(d, r, w, o, hidden, eps);
        else glue::residual_rmsnorm_kernel<__half, 4><<<rows, glue::NORM_THREADS, 0, st>>>(d, r, w, o, hidden, eps);
    }
    SKV_CUDA_TRY(cudaGetLastError());
    return SKV_OK;
}

int skv_silu_mul(const void* gate_up, void* out, int rows, int inter, int is_bf16, int device, void* stream) {
    if (!gate_up || !out) return fail(SKV_ERR_BAD_ARG, "skv_silu_mul: null pointer");
    if (rows <= 0 || inter <= 0 || inter % 8) return fail(SKV_ERR_BAD_ARG, "rows must be positive and inter a positive multiple of 8");
    if ((reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(out)) & 15)
        return fail(SKV_ERR_BAD_ARG, "skv_silu_mul: tensors must be 16-byte aligned");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(SKV_ERR_CUDA, "cannot switch to device %d", device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const long long items = (long long)rows * (inter / 8);
    const unsigned blocks = (unsigned)((items + 255) / 256);
    if (is_bf16) glue::silu_mul_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(static_cast<const uint16_t*>(gate_up), static_cast<uint16_t*>(out), rows, inter);
    else glue::silu_mul_kernel<__half><<<blocks, 256, 0, st>>>(static_cast<const uint16_t*>(gate_up), static_cast<uint16_t*>(out), rows, inter);
    SKV_CUDA_TRY(cudaGetLastError());
    return SKV_OK;
}

}  // extern "C"
