// Paged causal grouped-query attention, generic version: any head size up to 256 (16-byte loads where
// both head sizes are multiples of 16 bytes, element loads otherwise), values of another head size
// than queries and keys, any number of heads and groups, any page size, float32 or bfloat16 storage.  One kernel
// serves whole prompts, portions of prompts over a cached prefix, and single decoded tokens: the
// step's keys are in the cache before it runs, and a query at position p sees keys max(0, p-w+1)..p
// (w = window, 0 for all), which is the bottom-right-aligned causal rule of
// attention/torch_paged.py:36-45 (reference) expressed through positions.
//
// One warp per (token, query head).  Lane l takes keys lo+l, lo+l+32, ... and keeps its own running
// maximum, sum and output; lanes merge at the end.  The order of every sum depends only on the
// query's position, never on how the step was cut or what else is in the batch.  Softmax and both
// products accumulate in float32.
//
// Options of the score and of the weights (`AttentionExtras`), for designs that have them:
//   score(i, j) = q_i . k_j * scale - slopes[h] * (i - j) + head_bias[h]      (each term optional)
//   SIGMOID: the weight of a visible key is sigmoid(score), with no normalisation over the keys
//   gate: head h's output is multiplied by sigmoid(gate[t, h]) (one logit a token and head)
//   softcap c > 0: the scaled product becomes c tanh(q_i . k_j * scale / c) before the other terms
//   chunk n > 0: a query also sees no key before floor(i / n) * n (positions count from the request's first token)
//   out_f32: the output is written in float32 whatever the activation dtype
//   value_heads g > 0: the value pool holds g heads (a divisor of nkv), head h reads value head h / (nh / g): several
//     key heads, each with query heads of its own, over one set of values
#include "common.cuh"

struct AttentionExtras {
    const float* slopes;       // [nh] or null
    const float* head_bias;    // [nh] or null
    const void* gate;          // [tokens, nh] logits in the activation dtype, `gate_stride` elements a row, or null
    long long gate_stride;
    float softcap;             // 0: none
    int chunk;                 // 0: none
    int value_heads;           // 0: as many as key heads
    int out_f32;               // 1: `out` is float32 whatever the activation dtype
};

template <typename T>
struct Vec16;   // 16 bytes of T
template <>
struct Vec16<float> { static constexpr int N = 4; };
template <>
struct Vec16<__nv_bfloat16> { static constexpr int N = 8; };

template <typename T>
__device__ __forceinline__ void load16(const T* p, float (&out)[Vec16<T>::N]);
template <>
__device__ __forceinline__ void load16<float>(const float* p, float (&out)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}
template <>
__device__ __forceinline__ void load16<__nv_bfloat16>(const __nv_bfloat16* p, float (&out)[8]) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        out[2 * i] = f.x; out[2 * i + 1] = f.y;
    }
}

constexpr int WARPS = 4;

// queries: row t of `q` (`q_stride` elements a row), head h at h * hd; output [tokens, nh * vd]
template <typename T, int MAXHD, bool VEC, bool SIGMOID>
__global__ void __launch_bounds__(WARPS * 32)
paged_attention_generic_kernel(const T* __restrict__ q, long long q_stride, T* __restrict__ out,
                               const T* __restrict__ k_pool, const T* __restrict__ v_pool, KVGeometry geo, KVGeometry geo_v,
                               const int* __restrict__ block_table, int table_width, const int* __restrict__ positions,
                               const int* __restrict__ seq_of_token, int num_tokens, int nh, int nkv, int hd, int vd,
                               float scale, int window, AttentionExtras extras) {
    __shared__ float q_smem[WARPS][MAXHD];
    constexpr int VN = Vec16<T>::N;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)num_tokens * nh) return;
    const int t = (int)(item / nh), h = (int)(item % nh);
    const int seq = seq_of_token[t];
    T* o_ptr = out + ((long long)t * nh + h) * vd;
    if (seq < 0) return;                                      // padding row
    const int pos = positions[t];
    const int kvh = h / (nh / nkv);
    const T* q_ptr = q + (long long)t * q_stride + (long long)h * hd;
    for (int d = lane; d < hd; d += 32) q_smem[warp][d] = to_float<T>(q_ptr[d]) * scale;
    __syncwarp();

    float o[MAXHD];
#pragma unroll
    for (int d = 0; d < MAXHD; ++d) o[d] = 0.f;
    float m = -INFINITY, l = 0.f;
    const float slope = extras.slopes ? extras.slopes[h] : 0.f;
    const float bias = extras.head_bias ? extras.head_bias[h] : 0.f;

    int lo = window > 0 ? max(0, pos - window + 1) : 0;
    if (extras.chunk > 0) lo = max(lo, pos / extras.chunk * extras.chunk);
    const int vh = extras.value_heads > 0 ? h / (nh / extras.value_heads) : kvh;
    const float cap = extras.softcap, inv_cap = cap > 0.f ? 1.f / cap : 0.f;
    const long long head_off = geo.entry_offset + (long long)kvh * geo.page_tokens * hd;
    const long long head_off_v = geo_v.entry_offset + (long long)vh * geo.page_tokens * vd;
    const int* table = block_table + (long long)seq * table_width;
    for (int j = lo + lane; j <= pos; j += 32) {
        const int page = table[j / geo.page_tokens];
        if (page < 0 || page >= geo.num_pages) continue;      // a page given back (window) or a bad table
        const long long off = (long long)page * geo.page_stride + head_off + (long long)(j % geo.page_tokens) * hd;
        const T* kp = k_pool + off;
        float s = 0.f;
        if (VEC) {
#pragma unroll
            for (int d0 = 0; d0 < MAXHD; d0 += VN) {
                if (d0 < hd) {
                    float kv[VN];
                    load16<T>(kp + d0, kv);
#pragma unroll
                    for (int e = 0; e < VN; ++e) s = fmaf(q_smem[warp][d0 + e], kv[e], s);
                }
            }
        } else {
#pragma unroll 4
            for (int d = 0; d < hd; ++d) s = fmaf(q_smem[warp][d], to_float<T>(kp[d]), s);
        }
        if (cap > 0.f) s = cap * tanhf(s * inv_cap);
        s = s - slope * (float)(pos - j) + bias;
        float p;
        if (SIGMOID) {
            p = 1.f / (1.f + expf(-s));
        } else {
            if (s > m) {
                const float c = expf(m - s);                   // 0 on the first key (m = -inf)
                l *= c;
#pragma unroll
                for (int d = 0; d < MAXHD; ++d) o[d] *= c;
                m = s;
            }
            p = expf(s - m);
            l += p;
        }
        const T* vp = v_pool + (long long)page * geo_v.page_stride + head_off_v + (long long)(j % geo.page_tokens) * vd;
        if (VEC) {
#pragma unroll
            for (int d0 = 0; d0 < MAXHD; d0 += VN) {
                if (d0 < vd) {
                    float vv[VN];
                    load16<T>(vp + d0, vv);
#pragma unroll
                    for (int e = 0; e < VN; ++e) o[d0 + e] = fmaf(p, vv[e], o[d0 + e]);
                }
            }
        } else {
#pragma unroll
            for (int d = 0; d < MAXHD; ++d)
                if (d < vd) o[d] = fmaf(p, to_float<T>(vp[d]), o[d]);
        }
    }
    // merge the lanes
    float f = 1.f, inv = 1.f;
    if (!SIGMOID) {
        const float m_all = warp_max(m);
        f = (m == -INFINITY) ? 0.f : expf(m - m_all);
        const float l_all = warp_sum(l * f);
        inv = l_all > 0.f ? 1.f / l_all : 0.f;
    }
    if (extras.gate)
        inv /= 1.f + expf(-to_float<T>(((const T*)extras.gate)[(long long)t * extras.gate_stride + h]));
#pragma unroll
    for (int d = 0; d < MAXHD; ++d) {
        if (d < vd) {
            const float total = warp_sum(o[d] * f);
            if (lane == (d & 31)) {
                if (extras.out_f32) reinterpret_cast<float*>(out)[((long long)t * nh + h) * vd + d] = total * inv;
                else o_ptr[d] = from_float<T>(total * inv);
            }
        }
    }
}

template <typename T, int MAXHD>
static int launch(const void* q, long long q_stride, void* out, const void* k_pool, const void* v_pool, KVGeometry geo,
                  KVGeometry geo_v, const int* block_table, int table_width, const int* positions,
                  const int* seq_of_token, int num_tokens, int nh, int nkv, int hd, int vd, float scale, int window,
                  int sigmoid, AttentionExtras extras, cudaStream_t stream) {
    const long long items = (long long)num_tokens * nh;
    const unsigned blocks = (unsigned)((items + WARPS - 1) / WARPS);
    const int vn = Vec16<T>::N;
    // 16-byte loads need every row of keys and of values to start on a 16-byte boundary
    const bool vec = hd % vn == 0 && vd % vn == 0 && geo.page_stride % vn == 0 && geo.entry_offset % vn == 0 &&
                     geo_v.page_stride % vn == 0 && geo_v.entry_offset % vn == 0 && (uintptr_t)k_pool % 16 == 0 &&
                     (uintptr_t)v_pool % 16 == 0;
#define TS_ATTENTION_LAUNCH(V, S)                                                                                   \
    paged_attention_generic_kernel<T, MAXHD, V, S><<<blocks, WARPS * 32, 0, stream>>>(                              \
        (const T*)q, q_stride, (T*)out, (const T*)k_pool, (const T*)v_pool, geo, geo_v, block_table, table_width,   \
        positions, seq_of_token, num_tokens, nh, nkv, hd, vd, scale, window, extras)
    if (vec && sigmoid) TS_ATTENTION_LAUNCH(true, true);
    else if (vec) TS_ATTENTION_LAUNCH(true, false);
    else if (sigmoid) TS_ATTENTION_LAUNCH(false, true);
    else TS_ATTENTION_LAUNCH(false, false);
#undef TS_ATTENTION_LAUNCH
    TS_LAUNCH_CHECK("paged_attention_generic");
    return 0;
}

// Queries in a tensor of their own, values of head size `vd` in a pool with a geometry of its own; the options of
// the score and of the weights as arguments (`sigmoid` 1: sigmoid weights; null pointers: the term is absent).
TS_API int ts_paged_attention_scored(const void* q, long long q_stride, void* out, const void* k_pool, const void* v_pool,
                                     long long page_stride, long long entry_offset, long long v_page_stride,
                                     long long v_entry_offset, int page_tokens, int num_pages, const int* block_table,
                                     int table_width, const int* positions, const int* seq_of_token, int num_tokens,
                                     int nh, int nkv, int hd, int vd, float scale, int window, int dtype, int sigmoid,
                                     const float* slopes, const float* head_bias, const void* gate, long long gate_stride,
                                     float softcap, int chunk, int value_heads, int out_f32, cudaStream_t stream) {
    const AttentionExtras extras{slopes, head_bias, gate, gate_stride, softcap, chunk, value_heads, out_f32};
    TS_REQUIRE(softcap >= 0.f && chunk >= 0 && value_heads >= 0, "paged_attention: bad softcap, chunk or value heads");
    TS_REQUIRE(value_heads == 0 || (nkv % value_heads == 0 && nh % value_heads == 0),
               "paged_attention: %d value heads do not divide %d key heads", value_heads, nkv);
    TS_REQUIRE(num_tokens >= 0 && nh > 0 && nkv > 0, "paged_attention: bad sizes");
    TS_REQUIRE(nh % nkv == 0, "paged_attention: %d query heads are not a multiple of %d kv heads", nh, nkv);
    TS_REQUIRE(hd > 0 && hd <= 256 && vd > 0 && vd <= 256,
               "paged_attention: head sizes %d (keys) and %d (values) are not supported (up to 256)", hd, vd);
    TS_REQUIRE(page_tokens > 0 && table_width > 0 && window >= 0, "paged_attention: bad page geometry");
    if (num_tokens == 0) return 0;
    KVGeometry geo{page_stride, entry_offset, page_tokens, num_pages};
    KVGeometry geo_v{v_page_stride, v_entry_offset, page_tokens, num_pages};
    const int widest = hd > vd ? hd : vd;
#define TS_DISPATCH(TYPE)                                                                                          \
    if (widest <= 32) return launch<TYPE, 32>(q, q_stride, out, k_pool, v_pool, geo, geo_v, block_table, table_width, \
                                              positions, seq_of_token, num_tokens, nh, nkv, hd, vd, scale, window, sigmoid, extras, stream); \
    if (widest <= 64) return launch<TYPE, 64>(q, q_stride, out, k_pool, v_pool, geo, geo_v, block_table, table_width, \
                                              positions, seq_of_token, num_tokens, nh, nkv, hd, vd, scale, window, sigmoid, extras, stream); \
    if (widest <= 128) return launch<TYPE, 128>(q, q_stride, out, k_pool, v_pool, geo, geo_v, block_table, table_width, \
                                                positions, seq_of_token, num_tokens, nh, nkv, hd, vd, scale, window, sigmoid, extras, stream); \
    return launch<TYPE, 256>(q, q_stride, out, k_pool, v_pool, geo, geo_v, block_table, table_width, positions,      \
                             seq_of_token, num_tokens, nh, nkv, hd, vd, scale, window, sigmoid, extras, stream);
    if (dtype == TS_F32) { TS_DISPATCH(float) }
    if (dtype == TS_BF16) { TS_DISPATCH(__nv_bfloat16) }
#undef TS_DISPATCH
    return ts_fail("paged_attention: unknown dtype code %d", dtype);
}

// Softmax attention without further terms.
TS_API int ts_paged_attention_split(const void* q, long long q_stride, void* out, const void* k_pool, const void* v_pool,
                                    long long page_stride, long long entry_offset, long long v_page_stride,
                                    long long v_entry_offset, int page_tokens, int num_pages, const int* block_table,
                                    int table_width, const int* positions, const int* seq_of_token, int num_tokens,
                                    int nh, int nkv, int hd, int vd, float scale, int window, int dtype,
                                    cudaStream_t stream) {
    return ts_paged_attention_scored(q, q_stride, out, k_pool, v_pool, page_stride, entry_offset, v_page_stride,
                                     v_entry_offset, page_tokens, num_pages, block_table, table_width, positions,
                                     seq_of_token, num_tokens, nh, nkv, hd, vd, scale, window, dtype, 0, nullptr, nullptr,
                                     nullptr, 0, 0.f, 0, 0, 0, stream);
}

// Queries, keys and values of one head size in the columns [q | k | v] of one projection's output.
TS_API int ts_paged_attention_generic(const void* qkv, void* out, const void* k_pool, const void* v_pool,
                                      long long page_stride, long long entry_offset, int page_tokens, int num_pages,
                                      const int* block_table, int table_width, const int* positions,
                                      const int* seq_of_token, int num_tokens, int nh, int nkv, int hd, float scale,
                                      int window, int dtype, cudaStream_t stream) {
    TS_REQUIRE(hd > 0 && hd % 16 == 0 && hd <= 256,
               "paged_attention: head_dim %d is not supported (multiples of 16 up to 256)", hd);
    return ts_paged_attention_split(qkv, (long long)(nh + 2 * nkv) * hd, out, k_pool, v_pool, page_stride, entry_offset,
                                    page_stride, entry_offset, page_tokens, num_pages, block_table, table_width,
                                    positions, seq_of_token, num_tokens, nh, nkv, hd, hd, scale, window, dtype, stream);
}
