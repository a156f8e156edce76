/*
 * skv_b200.h -- C ABI of libskv_b200.so, the sm_100a (B200) kernels for the
 * long-context decode path: dense GQA split-KV decode attention, sparse decode
 * attention and fused KV eviction + quantisation.
 *
 * Conventions
 *   - every function returning int returns 0 on success and a negative SKV_ERR_*
 *     code otherwise; skv_last_error() then describes the failure (thread-local).
 *     Nothing throws across this boundary and nothing synchronises the stream
 *     unless its comment says so.
 *   - pointers named q/k/v/out/... are DEVICE pointers owned by the caller and
 *     borrowed for the duration of the asynchronous launch on `stream`
 *     (a cudaStream_t passed as void*); `device` is the CUDA ordinal they live on.
 *   - a workspace is caller-allocated device memory, 256-byte aligned, zero-filled
 *     ONCE before its first use; kernels leave it reusable.  One workspace must
 *     not be used by two launches that can overlap on the GPU.
 *   - strides are in ELEMENTS.
 *
 * Each entry point names the interface of the reference project
 * (SameerRajendra/LLM_Inference_Optimization) that it replaces.
 */
#ifndef SKV_B200_H
#define SKV_B200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SKV_OK 0
#define SKV_ERR_BAD_ARG (-1)
#define SKV_ERR_UNSUPPORTED (-2)
#define SKV_ERR_WORKSPACE (-3)
#define SKV_ERR_CUDA (-4)
#define SKV_ERR_DRIVER (-5)

/* KV cache element types */
#define SKV_KV_F16 0
#define SKV_KV_I8 1
#define SKV_KV_E4M3 2

/* bit in the workspace status word: a bounded wait inside a kernel ran out */
#define SKV_DEV_TIMEOUT 1

/* Replaces the c10::Error message carried by TORCH_CHECK in the reference launchers
 * (csrc/kernels/gqa_decode.cu:225-251). */
const char* skv_last_error(void);
int skv_abi_version(void);

/* Copies the status word at offset 0 of `workspace` to the host.  SYNCHRONISES `stream`.
 * No reference counterpart (the reference kernels have no device-side error reporting;
 * csrc/kernels/gqa_decode.cu:282-288 only checks the launch). */
int skv_workspace_status(const void* workspace, int device, void* stream, int* status_out);

/* ---- dense GQA decode --------------------------------------------------------------
 * Replaces launch_fused_gqa(Q, K, V, scale)  (csrc/kernels/gqa_decode.cu:218-290, bound as
 * sparse_kv._C.fused_gqa in csrc/pybind/bindings.cpp:29-30):
 *   out[b,hq,:] = softmax(scale * q[b,hq,:] . K[b,:,hq/(Hq/Hkv),:]^T) . V[b,:,hq/(Hq/Hkv),:]
 * q, out : [B, Hq, D] fp16 contiguous.   k, v : fp16, element (b,n,h,d) at
 * b*kv_stride_b + n*kv_stride_n + h*kv_stride_h + d  (the reference's [B,N,Hkv,D] layout is
 * kv_stride_b = N*Hkv*D, kv_stride_n = Hkv*D, kv_stride_h = D).  D is 64 or 128.
 * seq_lens : optional int32 [B] device array, tokens actually present per sequence (<= N).
 * kv_dtype : SKV_KV_F16 (k_scale / v_scale unused and may be NULL). */
size_t skv_gqa_decode_workspace_bytes(int B, int N, int Hq, int Hkv, int D, int device);
int skv_gqa_decode_splits(int B, int N, int Hq, int Hkv, int D, int device);
int skv_gqa_decode(const void* q, const void* k, const void* v, void* out,
                   void* workspace, size_t workspace_bytes,
                   int B, int N, int Hq, int Hkv, int D,
                   int kv_dtype, const float* k_scale, const float* v_scale,
                   long long kv_stride_b, long long kv_stride_n, long long kv_stride_h,
                   const int* seq_lens, float scale, int device, void* stream);
/* Pipeline depth (2..6 stages of 64 tokens) and CTAs per SM assumed when splitting the KV
 * length; process-wide.  No reference counterpart (the reference fixes TILE_SIZE/BLOCK_THREADS
 * at compile time, csrc/kernels/gqa_decode.cu:22-27). */
int skv_gqa_set_tuning(int stages, int ctas_per_sm);

/* Same computation as skv_gqa_decode (fp16 KV) for callers that cannot allocate device memory:
 * a server that has already handed every free byte of HBM to its KV page pool, or a C / Go host
 * with no torch allocator to borrow a workspace from.  NO COUNTERPART IN THE REFERENCE (its
 * launchers allocate through torch on every call, csrc/kernels/gqa_decode.cu:253).
 * The scratch is a fixed array inside the library: SKV_GQA_STATIC_SCRATCH_BYTES per GPU that loads
 * the library, kept until exit.  Problems whose skv_gqa_decode_workspace_bytes() is larger are
 * rejected with SKV_ERR_WORKSPACE.  The first call on a device looks the array's device address up
 * (make that call before any stream capture).  All calls on a GPU share the array: what must be
 * zero is cleared on `stream` before each launch, and calls that can overlap on one GPU race.
 * Calls no cudaMalloc / cudaFree / allocating library routine. */
#define SKV_GQA_STATIC_SCRATCH_BYTES (4u << 20)
int skv_gqa_decode_noalloc(const void* q, const void* k, const void* v, void* out,
                           int B, int N, int Hq, int Hkv, int D,
                           long long kv_stride_b, long long kv_stride_n, long long kv_stride_h,
                           const int* seq_lens, float scale, int device, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SKV_B200_H */
