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
/* OR-ed into kv_dtype of skv_gqa_decode_paged: the output tensor holds bf16 instead of fp16 elements. */
#define SKV_OUT_BF16 0x100
/* OR-ed into kv_dtype of skv_gqa_decode_paged, skv_quest_decode and skv_rope_quant_append: mixed-precision pages.  K stays 8-bit
 * (SKV_KV_I8 or SKV_KV_E4M3); V is 4-bit: code q = clamp(rne(v / scale), -7, 7) with scale = amax / 7 (1.0 for a zero
 * row), stored as the nibble q + 8, channel 2j in the low and 2j+1 in the high nibble of byte j (64 bytes per token).
 * The cache is one buffer of page records, [num_pages, Hkv, 25, 128] bytes: per (page, head) 16 rows of K codes,
 * 8 rows of V codes (two tokens per row), one row of 16 K scales then 16 V scales (fp32); pages hold 16 tokens.
 * Pass k_pool = record base, v_pool = base + 2048, k_scale_pool = base + 3072, v_scale_pool = base + 3136 (bytes),
 * pool strides (Hkv * 3200, 3200, 128) and scale strides (Hkv * 800, 800).  Up to 8 query heads per kv-head.
 * No reference counterpart. */
#define SKV_V_INT4 0x200
/* OR-ed into kv_dtype of skv_gqa_decode_paged: the kernel that precedes this call in the stream wrote nothing this call
 * reads except the query and each sequence's LAST token (position seq_lens[b] - 1: its code rows and scales), as
 * skv_rope_quant_append does.  The decode kernel, launched as a programmatic dependent, then streams every tile but the
 * one holding that token before the previous kernel has completed, and waits for it before reading that tile or the
 * query.  seq_lens and the page table must be older than the previous kernel.  Without the flag the kernel is ordered
 * like any other (or follows skv_gqa_set_early_kv). */
#define SKV_EARLY_EXCEPT_LAST 0x400

/* bit in the workspace status word: a bounded wait inside a kernel ran out */
#define SKV_DEV_TIMEOUT 1
/* bit in a status word: a page id read from the caller's page table lay outside [0, num_pages); the kernel read
 * page 0 in its place (decode) or stored nothing (append) instead of forming an address from it */
#define SKV_DEV_BAD_PAGE 2

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

/* ---- dense GQA decode over a paged 8-bit cache -----------------------------------
 * No reference counterpart (the reference reads an unpaged fp16 cache only, csrc/kernels/gqa_decode.cu:84-90, and
 * disables its INT8 path, csrc/kernels/kv_evict_quant.cu:294).
 *   out[b,hq,:] = softmax_t(scale * ks[t] * q[b,hq,:].kc[t,:]) . (vs[t] * vc[t,:])     kv-head = hq/(Hq/Hkv)
 * k_pool/v_pool : 1-byte codes (SKV_KV_I8 or SKV_KV_E4M3), element (page,h,slot,d) at
 *                 page*pool_stride_page + h*pool_stride_head + slot*pool_stride_slot + d, D = 128
 * k/v_scale_pool: fp32, element (page,h,slot) at page*scale_stride_page + h*scale_stride_head + slot
 * page_table    : int32 [B, max_pages] (physical page of tokens [i*page_size, (i+1)*page_size) of sequence b),
 *                 or NULL for page = b*max_pages + i (an unpaged [B,H,T,D] cache is page_size = T, max_pages = 1)
 * seq_lens      : int32 [B] or NULL (then every sequence holds N tokens).  N = longest length the launch must cover.
 * page_size is a multiple of 16.  Workspace: skv_gqa_decode_workspace_bytes(B, N, Hq, Hkv, D, device). */
int skv_gqa_decode_paged(const void* q, const void* k_pool, const void* v_pool,
                         const float* k_scale_pool, const float* v_scale_pool,
                         const int* page_table, const int* seq_lens, void* out,
                         void* workspace, size_t workspace_bytes,
                         int B, int N, int Hq, int Hkv, int D, int kv_dtype,
                         int page_size, int max_pages, int num_pages,
                         long long pool_stride_page, long long pool_stride_head, long long pool_stride_slot,
                         long long scale_stride_page, long long scale_stride_head,
                         float scale, int device, void* stream);
/* Ragged batches (seq_lens given): the host cannot read the lengths, so its split plan is sized for the longest
 * sequence the launch may hold.  on = 1 (default): when the batch has few (sequence, kv-head) pairs (at most 64
 * sequences and a quarter of the resident CTA slots) every CTA derives a work list of (sequence, split) items from
 * the real lengths -- one wave of CTAs of nearly equal length, none launched only to exit; on = 0: always the static
 * plan.  Same results either way.  Process-wide.  No reference counterpart. */
int skv_gqa_set_ragged_worklist(int on);
/* FP8 caches, at most 8 query heads per kv-head: mode 1 forces the kernel variant that fits two CTAs on an SM, 0 the
 * variant with one CTA per SM, -1 (default) lets the launcher choose by problem size.  Process-wide.  No reference
 * counterpart. */
int skv_gqa_set_q8_two_per_sm(int mode);
/* Ring depth of the 8-bit kernel (an even number of 17 KB stages in 4..12); process-wide.  No reference counterpart. */
int skv_gqa_set_q8_stages(int stages);
/* The decode kernels are launched with programmatic stream serialisation.  on = 0 (default): they wait for the
 * previous kernel of the stream before reading anything.  on = 1: K, V, the page table and seq_lens may be read
 * before that kernel has completed -- valid when it produces none of them (consecutive layers' decode calls over
 * caches written earlier); q, out and the workspace are always ordered.  Process-wide.  No reference counterpart. */
int skv_gqa_set_early_kv(int on);
/* Short contexts (up to 24 K tokens) of skv_gqa_decode: on = 1 (default) launches the splits of one (batch, kv-head)
 * as a thread-block cluster and sums them through distributed shared memory; on = 0 always uses the fp32 partials
 * in the workspace and the last-CTA ticket.  Results agree to fp32 rounding.  Process-wide.  No reference counterpart. */
int skv_gqa_set_cluster_combine(int on);

/* ---- Quest-style block-sparse decode over a paged 8-bit cache ----------------------
 * No reference counterpart (the reference scores blocks by the mean of q.k over an unpaged fp16 cache,
 * csrc/kernels/sparse_attention.cu:51-78).  Pools, scales, page_table, seq_lens as for skv_gqa_decode_paged.
 * skv_quest_build_meta: meta_out fp16 [B, Hkv, nb, 2, D], nb = skv_quest_num_blocks(N, block_size): channel-wise
 *   min ([..,0,:]) and max ([..,1,:]) of the dequantised keys (code * scale, fp32, rounded to fp16) of each block;
 *   a ragged last block covers its valid tokens only.
 * skv_quest_decode: block score for query head hq = scale * sum_d max(q_d*min_d, q_d*max_d) (fp32); the top_k_blocks
 *   best blocks per query head (ties: lower block id) among the blocks the sequence has; out[b,hq,:] = exact softmax
 *   attention over the tokens of those blocks (dequantised, fp32).  block_idx_out optional int32 [B,Hq,top_k_blocks],
 *   ascending, -1 padded.  D = 128, Hq/Hkv <= 8, top_k_blocks <= 256, top_k_blocks*block_size <= 2048.
 *   Workspace holds a status word (offset 0) and fp32 block scores [B,Hq,nb].
 *   kv_dtype | SKV_V_INT4: the cache is a buffer of mixed-precision page records (see SKV_V_INT4): v_pool rows are 64
 *   bytes of 4-bit codes; top_k_blocks*block_size <= 512 then.
 * num_pages: pages in the pools.  A page-table entry outside [0, num_pages) is never turned into an address: page 0 is
 *   read in its place and SKV_DEV_BAD_PAGE is set in the status word (skv_quest_build_meta: in *status, an optional
 *   int32 device word; skv_quest_decode: at offset 0 of the workspace, read with skv_workspace_status). */
int skv_quest_num_blocks(int N, int block_size);
/* on = 1 (default): skv_quest_decode scores the blocks on the tensor cores -- the bound sum_c max(q_c lo_c, q_c hi_c)
 * equals the dot product of (lo | hi) with (min(q, 0) | max(q, 0)) -- with the metadata streamed through a
 * shared-memory ring by TMA (up to 8 query heads per kv-head); on = 0: with the register-load kernel (also used for
 * larger groups).  Both sum the same exact products, in different orders.  Process-wide.  No reference counterpart. */
int skv_quest_set_ring_scores(int on);
/* on = 1: where it applies (tensor-core scoring on, Hq/Hkv <= 8, at most 2048 blocks per sequence)
 * skv_quest_decode is ONE kernel: thread-block clusters of Hq/Hkv CTAs (the query heads of a kv-head) stream the
 * kv-head's metadata together, score it for all heads and hand every head its scores through distributed shared memory,
 * then each CTA selects and attends; on = 0 (default): a scoring kernel followed by the select/attend kernel (the two
 * paths measure the same).  The scores are the same numbers either way.  Process-wide.  No reference counterpart. */
int skv_quest_set_fused(int on);
size_t skv_quest_workspace_bytes(int B, int Hq, int N, int block_size);
int skv_quest_build_meta(const void* k_pool, const float* k_scale_pool, const int* page_table, const int* seq_lens,
                         void* meta_out, int B, int N, int Hkv, int D, int kv_dtype, int block_size,
                         int page_size, int max_pages, int num_pages,
                         long long pool_stride_page, long long pool_stride_head, long long pool_stride_slot,
                         long long scale_stride_page, long long scale_stride_head, int* status, int device, void* stream);
int skv_quest_decode(const void* q, const void* k_pool, const void* v_pool,
                     const float* k_scale_pool, const float* v_scale_pool,
                     const int* page_table, const int* seq_lens, const void* meta,
                     void* out, int* block_idx_out, void* workspace, size_t workspace_bytes,
                     int B, int N, int Hq, int Hkv, int D, int kv_dtype,
                     int block_size, int top_k_blocks, int page_size, int max_pages, int num_pages,
                     long long pool_stride_page, long long pool_stride_head, long long pool_stride_slot,
                     long long scale_stride_page, long long scale_stride_head,
                     float scale, int device, void* stream);

/* ---- decode-step glue: RoPE + quantise + append -------------------------------------
 * Replaces the cache update the reference leaves to Hugging Face (DynamicCache.update concatenation and a
 * permute().contiguous() copy of the whole cache per layer and token, benchmarks/llama_integration_benchmark.py:173,
 * :302-303) and its RoPE call (:152-160).  qkv: [B, (Hq + 2 Hkv) * D] fp16 or bf16 (q heads, k heads, v heads);
 * q_out: [B, Hq, D] fp16 = rotate-half RoPE(q) at position seq_lens[b]; RoPE(k) and v are quantised per row
 * (scale = amax/448 for SKV_KV_E4M3, amax/127 for SKV_KV_I8; 1.0 for a zero row) and stored at token position
 * seq_lens[b] of sequence b in the paged pools (layout as for skv_gqa_decode_paged).  seq_lens is not modified; a
 * sequence whose position lies past its max_pages * page_size slots stores nothing.
 * meta (optional, else NULL): the fp16 [B,Hkv,meta_num_blocks,2,D] metadata of skv_quest_build_meta, whose block
 * containing the new token is updated with the dequantised new key (re-initialised when the token opens a block).
 * num_pages: pages in the pools; a table entry outside [0, num_pages) stores nothing and sets SKV_DEV_BAD_PAGE in
 * *status (optional int32 device word, else NULL).  D = 128. */
int skv_rope_quant_append(const void* qkv, int qkv_is_bf16, void* q_out, void* k_pool, void* v_pool,
                          float* k_scale_pool, float* v_scale_pool, const int* page_table, const int* seq_lens,
                          int B, int Hq, int Hkv, int D, int kv_dtype, int page_size, int max_pages,
                          long long pool_stride_page, long long pool_stride_head, long long pool_stride_slot,
                          long long scale_stride_page, long long scale_stride_head,
                          float rope_theta, void* meta, int meta_block_size, int meta_num_blocks,
                          int num_pages, int* status, int device, void* stream);

/* ---- token-sparse decode ----------------------------------------------------------
 * Replaces kv_evict_quant_forward(Q, K, V, top_k, use_int8=false)  (csrc/kernels/kv_evict_quant.cu:272-364,
 * bound in csrc/pybind/bindings.cpp:28) with the arithmetic of _reference_sparse_attention
 * (sparse_kv/attention.py:25-38): scores = scale * q.k over all T keys; only the top_k best keys and the
 * first sink_tokens positions take part in the softmax; out = sum w v.  The top-k is exact.
 * q [B,H,S,D], k/v [B,H,T,D] fp16 with element strides (channel contiguous, rows 16-byte aligned);
 * out [B,H,S,D] fp16 contiguous; topk_idx_out optional int32 [B,H,S,top_k], ascending, -1 padded.
 * D is 16, 32, 64, 128 or 256; min(top_k,T) + min(sink_tokens,T) <= 4096.  Workspace holds fp32 scores [B,H,S,T]. */
size_t skv_token_sparse_workspace_bytes(int B, int H, int S, int T);
/* on = 1 (default): decode-shaped calls (S = 1, D = 64 or 128) score the keys on the tensor cores, K streamed through a
 * shared-memory ring by TMA; on = 0: always the register-load kernel.  Both sum the same exact products in different
 * orders.  Process-wide.  The device status word (bit SKV_DEV_TIMEOUT) is at offset 0 of the workspace. */
int skv_token_sparse_set_mma_scores(int on);
/* on = 1 (default): the tensor-core scoring kernel cuts a row into chunks of unequal length (1.5 down to 0.5 times the
 * mean), so that the CTAs' per-chunk candidate selections are spread over time instead of coinciding wave after wave;
 * on = 0: equal chunks.  Same results either way.  Process-wide.  No reference counterpart. */
int skv_token_sparse_set_stagger(int on);
int skv_token_sparse_decode(const void* q, const void* k, const void* v, void* out, int* topk_idx_out,
                            void* workspace, size_t workspace_bytes, int B, int H, int S, int T, int D,
                            long long q_stride_b, long long q_stride_h, long long q_stride_s,
                            long long kv_stride_b, long long kv_stride_h, long long kv_stride_t,
                            int top_k, int sink_tokens, float scale, int device, void* stream);

/* ---- block-sparse decode, block-mean rule -----------------------------------------
 * Replaces sparse_attention_forward(Q, K, V, block_size, top_k_blocks)  (csrc/kernels/sparse_attention.cu:178-244,
 * kernel :26-175; bound in csrc/pybind/bindings.cpp:27; same arithmetic as jax_ref/sparse_attention_pallas.py:52-136):
 *   s_j = scale * mean_{t in block j} q.k_t;  top_k_blocks best blocks (ties: lower block);  w = softmax(s_top);
 *   out = sum_j w_j * mean_{t in block j} v_t.   The ragged last block uses its own token count.
 * q [B,H,D] (the reference's [B,H,1,D]), k/v [B,H,T,D] fp16 with element strides; out [B,H,D] fp16 contiguous;
 * block_idx_out optional int32 [B,H,top_k_blocks], ascending, -1 padded (the reference computes and drops it,
 * sparse_attention.cu:213-215,243).  D is 16, 32, 64, 128 or 256; min(top_k_blocks, nb) <= 4096.
 * Workspace holds fp32 block scores [B,H,nb]. */
size_t skv_block_sparse_workspace_bytes(int B, int H, int T, int block_size);
/* on = 1 (default): with D = 64 or 128 and a block size that is a multiple of 16 the block scores are computed on the
 * tensor cores (the mean of q . k_t over a block is the sum of its tokens' scores over their count), K streamed through
 * a shared-memory ring by TMA; on = 0: always the register-load kernel.  Process-wide.  The device status word (bit
 * SKV_DEV_TIMEOUT) is at offset 0 of the workspace. */
int skv_block_sparse_set_mma_scores(int on);
int skv_block_sparse_decode(const void* q, const void* k, const void* v, void* out, int* block_idx_out,
                            void* workspace, size_t workspace_bytes, int B, int H, int T, int D,
                            long long q_stride_b, long long q_stride_h,
                            long long kv_stride_b, long long kv_stride_h, long long kv_stride_t,
                            int block_size, int top_k_blocks, float scale, int device, void* stream);

/* ---- fused KV eviction + quantisation ----------------------------------------------
 * Replaces fused_kv_evict / _reference_eviction (sparse_kv/eviction.py:12-27, :30-44): per (b,h) keep the
 * `budget` highest-scoring tokens (scores fp32 [B,H,T] contiguous) plus the last `recent` positions, gather
 * their K and V rows and quantise them.  keep = skv_kv_evict_keep_count(T, budget, recent).
 *   idx_out      int32 [B,H,keep]: kept positions, ascending (order 0) or by descending score (order 1,
 *                the order torch.topk returns; equal scores: lower position first)
 *   k_out/v_out  [B,H,keep,D]: fp16 rows (quant_mode 0), int8 codes (1), e4m3 codes (2), or the
 *                reference's unscaled int8 cast (3; sparse_kv/eviction.py:41-43)
 *   k/v_scale_out fp32 [B,H,keep], required for modes 1 and 2:
 *                mode 1: scale = amax/127 (1.0 if the row is zero), code = clamp(rint(x/scale), -127, 127)
 *                mode 2: scale = amax/448 (1.0 if zero),            code = e4m3_rne_satfinite(x/scale)
 * k_cache/v_cache fp16 [B,H,T,D] with element strides.  D is 16, 32, 64, 128 or 256, keep <= 8192. */
int skv_kv_evict_keep_count(int T, int budget, int recent);
/* on = 1: position-order evictions of rows with at most 32768 competing scores and D = 64 or 128 run as ONE launch
 * (a 4-CTA cluster per (b,h) selects, then gathers and quantises its own head's rows); on = 0 (default): selection
 * and gather run as two launches, the second a programmatic dependent of the first -- measured a few microseconds
 * faster at B*H = 32 because the gather then spreads over every SM.  Same results either way; process-wide.
 * No reference counterpart. */
int skv_kv_evict_set_fused(int on);
int skv_kv_evict_quant(const void* k_cache, const void* v_cache, const float* scores, int* idx_out,
                       void* k_out, void* v_out, float* k_scale_out, float* v_scale_out,
                       int B, int H, int T, int D,
                       long long kv_stride_b, long long kv_stride_h, long long kv_stride_t,
                       int budget, int recent, int quant_mode, int order, int device, void* stream);

/* skv_gqa_decode (fp16 KV) that also ACCUMULATES the attention mass of every cached token:
 *   mass[b, hkv, t] += sum over the query heads hq of kv-head hkv of softmax_t(scale * q[b,hq] . k[b,t,hkv])
 * mass: fp32 [B, Hkv, N], read-modify-write for t < seq_lens[b] (N without seq_lens).  This is the per-token
 * importance score that the reference's fused_kv_evict takes as `scores` (sparse_kv/eviction.py:12-22) and leaves
 * to its caller to produce; summed over decode steps it drives skv_kv_evict_quant.  The decode kernel stores its
 * scaled scores (fp32 [B,Hq,N]) and each head's final softmax maximum and denominator in the workspace, and a
 * second small kernel turns them into probabilities.  Workspace: skv_gqa_decode_mass_workspace_bytes(). */
size_t skv_gqa_decode_mass_workspace_bytes(int B, int N, int Hq, int Hkv, int D, int device);
int skv_gqa_decode_mass(const void* q, const void* k, const void* v, void* out, float* mass,
                        void* workspace, size_t workspace_bytes, int B, int N, int Hq, int Hkv, int D,
                        long long kv_stride_b, long long kv_stride_n, long long kv_stride_h,
                        const int* seq_lens, float scale, int device, void* stream);

/* Same computation as skv_gqa_decode (fp16 KV) for callers that cannot allocate device memory:
 * a server that has already handed every free byte of HBM to its KV page pool, or a C / Go host
 * with no torch allocator to borrow a workspace from.  NO COUNTERPART IN THE REFERENCE (its
 * launchers allocate through torch on every call, csrc/kernels/gqa_decode.cu:253).
 * The scratch is a fixed array inside the library: SKV_GQA_STATIC_SCRATCH_BYTES per GPU that loads
 * the library, kept until exit.  Problems whose skv_gqa_decode_workspace_bytes() is larger are
 * rejected with SKV_ERR_WORKSPACE.  The first call on a device looks the array's device address up
 * (make that call before any stream capture; made during a capture it returns SKV_ERR_CUDA).  All calls on a GPU share the array: what must be
 * zero is cleared on `stream` before each launch, and calls that can overlap on one GPU race.
 * Calls no cudaMalloc / cudaFree / allocating library routine. */
#define SKV_GQA_STATIC_SCRATCH_BYTES (4u << 20)
int skv_gqa_decode_noalloc(const void* q, const void* k, const void* v, void* out,
                           int B, int N, int Hq, int Hkv, int D,
                           long long kv_stride_b, long long kv_stride_n, long long kv_stride_h,
                           const int* seq_lens, float scale, int device, void* stream);
/* Reads the status word of that built-in array on `device` (SKV_DEV_TIMEOUT when a bounded wait inside the kernel
 * ran out; the per-call clearing leaves this word alone, so a bit stays set until the process ends).  SYNCHRONISES
 * `stream`.  Allocates nothing.  No counterpart in the reference. */
int skv_gqa_decode_noalloc_status(int device, void* stream, int* status_out);

/* ---- decode-step glue around the attention call -------------------------------------
 * The reference runs Hugging Face's LlamaRMSNorm / LlamaMLP modules here (the model it patches,
 * benchmarks/llama_integration_benchmark.py:266-279); with 16 rows per step those are launch-bound.
 * skv_residual_rmsnorm: resid[r,:] <- round(resid + delta) when delta is non-null (in place), then
 *   out[r,:] = round(resid * rsqrt(mean(resid^2) + eps) * weight); [rows, hidden] row-major, hidden % 8 == 0,
 *   hidden <= 8192, fp16 (is_bf16 = 0) or bf16 elements, 16-byte aligned.
 * skv_silu_mul: out[r,c] = round(round(silu(gate_up[r,c])) * gate_up[r,inter+c]); gate_up [rows, 2*inter], out [rows, inter]. */
int skv_residual_rmsnorm(const void* delta, void* resid, const void* weight, void* out, int rows, int hidden, float eps,
                         int is_bf16, int device, void* stream);
int skv_silu_mul(const void* gate_up, void* out, int rows, int inter, int is_bf16, int device, void* stream);

/* ---- decode-step projections: skinny GEMM ------------------------------------------------------------
 * The reference runs the q/k/v, o, gate/up and down projections as Hugging Face nn.Linear modules (the model it
 * patches, benchmarks/llama_integration_benchmark.py:266-279).  out[M,N] = x[M,K] . w[K,N], all row-major and
 * contiguous, fp16 (is_bf16 = 0) or bf16 elements, fp32 accumulation; 1 <= M <= 16, K % 32 == 0, N % 64 == 0
 * (other shapes: SKV_ERR_UNSUPPORTED, and skv_skinny_gemm_workspace_bytes returns 0).  The workspace is zero-filled
 * once before its first use; its status word (offset 0) is read with skv_workspace_status.  The result does not
 * depend on the order in which CTAs finish.  skv_skinny_gemm_set_min_blocks (tuning, process-wide): the fewest
 * 16 KB blocks of w a CTA streams on small problems (default 16); it changes the workspace size of a shape. */
int skv_skinny_gemm_set_min_blocks(int blocks);
size_t skv_skinny_gemm_workspace_bytes(int M, int K, int N, int device);
int skv_skinny_gemm(const void* x, const void* w, void* out, void* workspace, size_t workspace_bytes,
                    int M, int K, int N, int is_bf16, int device, void* stream);

/* ---- tensor-parallel decode step: all-reduce + residual add + RMSNorm in one kernel over peer memory ----
 * No reference counterpart (the reference is single-GPU).  Every rank passes the same arrays, indexed by rank:
 * peer_partials[r] = device address, valid on THIS GPU, of rank r's [rows, hidden] partial sum (peer-mapped /
 * symmetric memory); peer_flags[r] = rank r's flag array of 8 uint32 (zero before the first call, written by
 * peers).  sync_words: 4 zero-initialised uint32 in this rank's own memory ([0] epoch, [1] ticket, [2] status).
 * The kernel tells the peers that this rank's partial is complete, waits (at most max_spins polls per peer, then
 * status |= 1 (SKV_DEV_TIMEOUT) and nothing is stored; while the status word is non-zero later calls
 * fail at once instead of waiting) until every peer has said the same, and computes
 *   resid <- round(resid + round(sum_r partial_r)),  out <- round(resid * rsqrt(mean(resid^2) + eps) * weight).
 * Consecutive calls must alternate between two partial buffers.  world in {1,2,4,8}; fp16 or bf16. */
int skv_allreduce_residual_rmsnorm(const void* const* peer_partials, void* const* peer_flags, void* sync_words,
                                   void* resid, const void* weight, void* out, int rows, int hidden, float eps,
                                   int is_bf16, int rank, int world, unsigned max_spins, int device, void* stream);
/* Push variant of the same step: instead of announcing its partial and letting the peers read it (two NVLink traversals
 * in sequence), every rank WRITES its partial row into a receive region of every peer, in 8-byte words that carry 4 bytes
 * of the partial and the 32-bit epoch of the call -- the data is its own flag, no fence is needed, one traversal.  The
 * kernel then polls its own receive region (bounded like the waits above) and sums the ranks' rows in rank order.
 * partial: this rank's [rows, hidden] partial sum in its own memory.  peer_recv[r]: device address, valid on THIS GPU,
 * of rank r's receive region for this call: world * rows * hidden * 4 bytes ([source rank][rows][hidden / 2] words),
 * zero-filled before the first call; consecutive calls must alternate between two regions.  hidden <= 4096.
 * sync_words and every other argument as above.  No reference counterpart. */
int skv_allreduce_residual_rmsnorm_push(const void* partial, void* const* peer_recv, void* sync_words, void* resid,
                                        const void* weight, void* out, int rows, int hidden, float eps, int is_bf16,
                                        int rank, int world, unsigned max_spins, int device, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SKV_B200_H */
