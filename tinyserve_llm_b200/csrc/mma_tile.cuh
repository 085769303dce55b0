// Pieces the tensor-core attention kernels (mma.sync m16n8k16, bfloat16 operands, float32 sums) share:
// cp.async copies, ldmatrix and mma wrappers, tiles in shared memory whose 16-byte chunks are
// XOR-swizzled by the row, and the address of a key or value row in the paged cache.
#pragma once

#include "common.cuh"

static __device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

static __device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const int bytes = valid ? 16 : 0;                       // 0: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(smem)), "l"(gmem), "r"(bytes));
}
static __device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
static __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

static __device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
static __device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
static __device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
static __device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// A tile in shared memory: ROWS rows of HD bfloat16, 16-byte chunks XOR-swizzled by the row.
template <int HD>
static __device__ __forceinline__ __nv_bfloat16* tile_at(__nv_bfloat16* tile, int row, int chunk) {
    return tile + row * HD + ((chunk ^ (row & 7)) << 3);
}

// Loads `rows` rows of HD bfloat16 (row r from src + r * src_stride) into a swizzled tile with the
// `nthreads` threads given; rows >= valid_rows are zero-filled.
template <int HD>
static __device__ __forceinline__ void load_tile(__nv_bfloat16* tile, const __nv_bfloat16* src, long long src_stride,
                                          int rows, int valid_rows, int tid, int nthreads) {
    constexpr int CHUNKS = HD / 8;
    for (int i = tid; i < rows * CHUNKS; i += nthreads) {
        const int r = i / CHUNKS, c = i % CHUNKS;
        const bool ok = r < valid_rows;
        cp_async16(tile_at<HD>(tile, r, c), src + (ok ? (long long)r * src_stride + c * 8 : 0), ok);
    }
}

// Address of key (or value) row `key` of kv head `kvh` of the request whose table is given; null if
// the page was given back.
template <int HD>
static __device__ __forceinline__ const __nv_bfloat16* kv_row_of_page(const __nv_bfloat16* pool, const KVGeometry& geo, int page,
                                                               int kvh, int key) {
    if (page < 0 || page >= geo.num_pages) return nullptr;
    return pool + (long long)page * geo.page_stride + geo.entry_offset + ((long long)kvh * geo.page_tokens + key % geo.page_tokens) * HD;
}
template <int HD>
static __device__ __forceinline__ const __nv_bfloat16* kv_row(const __nv_bfloat16* pool, const KVGeometry& geo,
                                                       const int* table, int kvh, int key) {
    return kv_row_of_page<HD>(pool, geo, table[key / geo.page_tokens], kvh, key);
}

