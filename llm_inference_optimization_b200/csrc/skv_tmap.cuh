// Host-side construction of TMA tensor maps over a KV cache.
//
// The caches this library reads are addressed as (batch, token, kv-head, channel)
// with arbitrary element strides for batch / token / head (channel is contiguous),
// which covers both layouts the reference uses: [B, N, Hkv, D] for the dense
// decode entry point and [B, H, T, D] for the sparse entry points.
//
// A 16-bit cache row of D channels is exposed to TMA as D/64 "halves" of 64
// channels (128 bytes) so that each half lands in shared memory as a
// [tile_tokens][64] block with the 128-byte swizzle, which ldmatrix then reads
// without bank conflicts.  Tensor dimensions above the innermost are sorted by
// stride; the position each logical dimension ended up in is returned so the
// kernel can place its coordinates.
#pragma once

#include <algorithm>

#include "skv_common.cuh"

namespace skv {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// A decode step encodes the same maps again and again (one call per layer and token over caches that do not move),
// so the last few encodings are kept per host thread, keyed by every argument that goes into them.
template <typename Pos>
struct TmapCache {
    static constexpr int SLOTS = 128;
    struct Entry {
        long long key[12];
        CUtensorMap map;
        Pos pos;
        bool valid = false;
    };
    Entry e[SLOTS];
    const Entry* find(const long long (&key)[12]) const {
        const Entry& x = e[slot(key)];
        if (!x.valid) return nullptr;
        for (int i = 0; i < 12; ++i)
            if (x.key[i] != key[i]) return nullptr;
        return &x;
    }
    void put(const long long (&key)[12], const CUtensorMap& m, const Pos& pos) {
        Entry& x = e[slot(key)];
        for (int i = 0; i < 12; ++i) x.key[i] = key[i];
        x.map = m;
        x.pos = pos;
        x.valid = true;
    }
    static int slot(const long long (&key)[12]) {
        unsigned long long h = 1469598103934665603ull;
        for (int i = 0; i < 12; ++i) h = (h ^ (unsigned long long)key[i]) * 1099511628211ull;
        return (int)((h >> 20) % SLOTS);
    }
};

// Where each logical coordinate sits among the tensor map's dimensions 1..4
// (dimension 0 is always the contiguous channel run).
struct KvMapPos {
    int half, tok, head, batch;
};

// Build the map for a cache with `elem_bytes`-wide elements.
//   inner_elems : channels per innermost run (64 for 16-bit, D for 8-bit)
//   n_half      : D / inner_elems
//   strides in ELEMENTS.
inline int make_kv_tmap(CUtensorMap* out, KvMapPos* pos, const void* base, int elem_bytes, int inner_elems,
                        int n_half, long long B, long long N, long long Hkv, long long stride_b, long long stride_n,
                        long long stride_h, int tile_tokens) {
    static thread_local TmapCache<KvMapPos> cache;
    const long long key[12] = {(long long)reinterpret_cast<uintptr_t>(base), elem_bytes, inner_elems, n_half, B, N, Hkv,
                               stride_b, stride_n, stride_h, tile_tokens, 0};
    if (const auto* hit = cache.find(key)) {
        *out = hit->map;
        *pos = hit->pos;
        return SKV_OK;
    }
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return fail(SKV_ERR_DRIVER, "cuTensorMapEncodeTiled entry point not available");
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0)
        return fail(SKV_ERR_BAD_ARG, "KV base pointer must be 16-byte aligned for TMA");

    struct Dim {
        int logical;  // 1 half, 2 token, 3 head, 4 batch
        unsigned long long size, stride_bytes;
        unsigned box;
    } d[4] = {
        {1, (unsigned long long)n_half, (unsigned long long)inner_elems * elem_bytes, 1u},
        {2, (unsigned long long)N, (unsigned long long)stride_n * elem_bytes, (unsigned)tile_tokens},
        {3, (unsigned long long)Hkv, (unsigned long long)stride_h * elem_bytes, 1u},
        {4, (unsigned long long)B, (unsigned long long)stride_b * elem_bytes, 1u},
    };
    for (auto& x : d) {
        if (x.size == 1 && (x.stride_bytes == 0 || (x.stride_bytes & 15))) x.stride_bytes = 16;  // unused stride
        if (x.stride_bytes == 0 || (x.stride_bytes & 15))
            return fail(SKV_ERR_BAD_ARG, "KV stride of %llu bytes is not a positive multiple of 16", x.stride_bytes);
    }
    std::stable_sort(d, d + 4, [](const Dim& a, const Dim& b) { return a.stride_bytes < b.stride_bytes; });

    cuuint64_t gdim[5] = {(cuuint64_t)inner_elems, d[0].size, d[1].size, d[2].size, d[3].size};
    cuuint64_t gstr[4] = {d[0].stride_bytes, d[1].stride_bytes, d[2].stride_bytes, d[3].stride_bytes};
    cuuint32_t box[5] = {(cuuint32_t)inner_elems, d[0].box, d[1].box, d[2].box, d[3].box};
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    for (int i = 0; i < 4; ++i) {
        int p = i + 1;
        switch (d[i].logical) {
            case 1: pos->half = p; break;
            case 2: pos->tok = p; break;
            case 3: pos->head = p; break;
            default: pos->batch = p; break;
        }
    }
    CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    int inner_bytes = inner_elems * elem_bytes;
    CUtensorMapSwizzle sw = inner_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                          : inner_bytes == 64  ? CU_TENSOR_MAP_SWIZZLE_64B
                                               : CU_TENSOR_MAP_SWIZZLE_NONE;
    CUresult r = enc(out, dt, 5, const_cast<void*>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(SKV_ERR_DRIVER, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    cache.put(key, *out, *pos);
    return SKV_OK;
}

// Map over a row-major 16-bit matrix [rows, cols] with `ld` elements between rows: box = box_rows x box_cols, with
// box_cols 64 (128-byte rows, 128-byte swizzle) or 32 (64-byte rows, 64-byte swizzle).  Coordinates: (column, row).
// Rows past `rows` and columns past `cols` read as zero.
inline int make_matrix_tmap(CUtensorMap* out, const void* base, long long rows, long long cols, long long ld,
                            int box_rows, int box_cols, bool bf16) {
    static thread_local TmapCache<int> cache;
    const long long key[12] = {(long long)reinterpret_cast<uintptr_t>(base), rows, cols, ld, box_rows, bf16 ? 1 : 0, box_cols, 0, 0, 0, 0, 2};
    if (const auto* hit = cache.find(key)) {
        *out = hit->map;
        return SKV_OK;
    }
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return fail(SKV_ERR_DRIVER, "cuTensorMapEncodeTiled entry point not available");
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (ld * 2) % 16 != 0)
        return fail(SKV_ERR_BAD_ARG, "matrix base and row pitch must be 16-byte aligned for TMA");
    cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t gstr[1] = {(cuuint64_t)ld * 2};
    if (box_cols != 64 && box_cols != 32) return fail(SKV_ERR_BAD_ARG, "matrix box must be 32 or 64 elements wide");
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(out, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                     const_cast<void*>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     box_cols == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(SKV_ERR_DRIVER, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    cache.put(key, *out, 0);
    return SKV_OK;
}

// Where each logical coordinate of a paged 8-bit pool sits among tensor-map dimensions 1..3.
struct PoolMapPos {
    int slot, head, page;
};

// Map over a pool of 1-byte codes addressed as (page, head, slot, channel): rows of D bytes,
// box = `box_slots` consecutive slots of one (page, head), 128-byte swizzle (D must be 128).
inline int make_pool_tmap(CUtensorMap* out, PoolMapPos* pos, const void* base, int D, long long num_pages,
                          long long Hkv, long long page_size, long long stride_page, long long stride_head,
                          long long stride_slot, int box_slots) {
    static thread_local TmapCache<PoolMapPos> cache;
    const long long key[12] = {(long long)reinterpret_cast<uintptr_t>(base), D, num_pages, Hkv, page_size, stride_page,
                               stride_head, stride_slot, box_slots, 0, 0, 1};
    if (const auto* hit = cache.find(key)) {
        *out = hit->map;
        *pos = hit->pos;
        return SKV_OK;
    }
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return fail(SKV_ERR_DRIVER, "cuTensorMapEncodeTiled entry point not available");
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0)
        return fail(SKV_ERR_BAD_ARG, "pool base pointer must be 16-byte aligned for TMA");
    struct Dim {
        int logical;  // 1 slot, 2 head, 3 page
        unsigned long long size, stride_bytes;
        unsigned box;
    } d[3] = {
        {1, (unsigned long long)page_size, (unsigned long long)stride_slot, (unsigned)box_slots},
        {2, (unsigned long long)Hkv, (unsigned long long)stride_head, 1u},
        {3, (unsigned long long)num_pages, (unsigned long long)stride_page, 1u},
    };
    for (auto& x : d) {
        if (x.size == 1 && (x.stride_bytes == 0 || (x.stride_bytes & 15))) x.stride_bytes = 16;
        if (x.stride_bytes == 0 || (x.stride_bytes & 15))
            return fail(SKV_ERR_BAD_ARG, "pool stride of %llu bytes is not a positive multiple of 16", x.stride_bytes);
    }
    std::stable_sort(d, d + 3, [](const Dim& a, const Dim& b) { return a.stride_bytes < b.stride_bytes; });
    // Rows are declared as D/4 32-bit words rather than D bytes: the copy is byte-identical (the 128-byte
    // swizzle works on addresses), and wider elements keep the TMA unit's per-element work low.
    cuuint64_t gdim[4] = {(cuuint64_t)D / 4, d[0].size, d[1].size, d[2].size};
    cuuint64_t gstr[3] = {d[0].stride_bytes, d[1].stride_bytes, d[2].stride_bytes};
    cuuint32_t box[4] = {(cuuint32_t)D / 4, d[0].box, d[1].box, d[2].box};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    for (int i = 0; i < 3; ++i) {
        const int p = i + 1;
        if (d[i].logical == 1) pos->slot = p; else if (d[i].logical == 2) pos->head = p; else pos->page = p;
    }
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, const_cast<void*>(base), gdim, gstr, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(SKV_ERR_DRIVER, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    cache.put(key, *out, *pos);
    return SKV_OK;
}

}  // namespace skv
