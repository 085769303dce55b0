// Attention whose keys and values are up-projections of one cached latent per token, plus one
// rotated key part that all heads share.  Per token the cache holds a row [c | k_rot] of
// rank + rot_dim elements (one "kv head", no value pool): c is the normed latent, k_rot the rotated part.
//
// With K_h = W_uk,h c and V_h = W_uv,h c the score of head h is
//   q_flat,h . (W_uk,h c) + q_rot,h . k_rot  =  (W_uk,h^T q_flat,h) . c + q_rot,h . k_rot
// so the kernel works on the latent itself: the caller folds W_uk into the query (q_lat = W_uk^T q_flat,
// a batched product), the kernel takes scores against [c | k_rot], softmax over the visible keys, the
// weighted sum of c, and the caller applies W_uv to that sum.  Nothing of a head's keys or values is
// ever materialised, for prompts and for decoding alike.
//
// ts_latent_prepare: per token, norms the query latent and the key/value latent (plain weights),
// rotates the shared key part (rotate-half, angle = position * freq[i], float32) and stores [c | k_rot]
// into the token's slot of the paged cache.
// ts_latent_attention: bfloat16 with sizes it takes runs on the tensor-core kernel of attention_latent_mma.cu;
// float32 and all other sizes here: one CTA per token and group of up to 8 heads (a warp a head).  Keys come in
// tiles of 32 into shared memory as float32, shared by the heads; lane j scores key j of the tile, the
// online softmax runs across the warp, and lane l accumulates channels l, l + 32, ... of the output.
// A query at position p sees keys max(0, p - window + 1) .. p (window 0: all).  The order of every sum
// depends on the query's position only.  In a step of few tokens (decoding) a token's keys are split over
// several CTAs, 128 keys each counted from the window's first key, and a second kernel merges the
// partial results in key order: again nothing depends on the rest of the batch.
#include "common.cuh"

bool ts_latent_mma_supported(int rank, int rot);
int ts_latent_attention_mma_launch(const float* q_lat, long long ql_t, long long ql_h, const void* q, long long q_stride,
                                   int q_head_width, int q_rot_offset, const float* freq, const void* k_pool,
                                   KVGeometry geo, const int* block_table, int table_width, const int* positions,
                                   const int* seq_of_token, void* out, int num_tokens, int heads, int rank, int rot,
                                   float scale, int window, int split_keys, int splits, float* partial, cudaStream_t stream);

constexpr int LA_WARPS = 8;
constexpr int LA_KEYS = 32;
constexpr int LA_SPLIT = 128;       // keys of one CTA when a small step's keys are split over several

template <typename T>
__global__ void latent_prepare_kernel(const T* __restrict__ y, long long y_stride, int q_rank, int rank, int rot,
                                      const float* __restrict__ wq, const float* __restrict__ wkv, float eps,
                                      const float* __restrict__ freq, const int* __restrict__ positions,
                                      const int* __restrict__ seq_of_token, T* __restrict__ cq, T* k_pool, KVGeometry geo,
                                      const int* __restrict__ block_table, int table_width, int writes) {
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const int seq = seq_of_token[t];
    if (seq < 0) return;
    const T* row = y + (long long)t * y_stride;
    float acc = 0.f;
    if (q_rank > 0) {                                     // q_rank 0: the queries have no latent of their own
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x) { const float x = to_float<T>(row[i]); acc += x * x; }
        const float inv_q = 1.f / sqrtf(block_sum(acc, scratch) / (float)q_rank + eps);
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
            cq[(long long)t * q_rank + i] = from_float<T>(to_float<T>(row[i]) * inv_q * wq[i]);
        __syncthreads();
    }
    if (!writes) return;
    acc = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) { const float x = to_float<T>(row[q_rank + i]); acc += x * x; }
    const float inv_c = 1.f / sqrtf(block_sum(acc, scratch) / (float)rank + eps);
    const int pos = positions[t];
    const int page = block_table[(long long)seq * table_width + pos / geo.page_tokens];
    if (page < 0 || page >= geo.num_pages) return;
    T* dst = k_pool + (long long)page * geo.page_stride + geo.entry_offset + (long long)(pos % geo.page_tokens) * (rank + rot);
    for (int i = threadIdx.x; i < rank; i += blockDim.x)
        dst[i] = from_float<T>(to_float<T>(row[q_rank + i]) * inv_c * wkv[i]);
    const int half = rot / 2;
    const T* kr = row + q_rank + rank;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * freq[i], &sn, &cs);
        const float u = to_float<T>(kr[i]), v = to_float<T>(kr[i + half]);
        dst[rank + i] = from_float<T>(u * cs - v * sn);
        dst[rank + i + half] = from_float<T>(v * cs + u * sn);
    }
}

TS_API int ts_latent_prepare(const void* y, long long y_stride, int q_rank, int rank, int rot, const float* wq,
                             const float* wkv, float eps, const float* freq, const int* positions,
                             const int* seq_of_token, void* cq, void* k_pool, long long page_stride, long long entry_offset,
                             int page_tokens, int num_pages, const int* block_table, int table_width, int writes,
                             int num_tokens, int dtype, cudaStream_t stream) {
    TS_REQUIRE(q_rank >= 0 && rank > 0 && rot >= 0 && rot % 2 == 0, "latent_prepare: bad sizes");
    TS_REQUIRE(page_tokens > 0 && table_width > 0, "latent_prepare: bad page geometry");
    if (num_tokens == 0) return 0;
    KVGeometry geo{page_stride, entry_offset, page_tokens, num_pages};
    if (dtype == TS_F32)
        latent_prepare_kernel<float><<<num_tokens, 128, 0, stream>>>((const float*)y, y_stride, q_rank, rank, rot, wq, wkv,
            eps, freq, positions, seq_of_token, (float*)cq, (float*)k_pool, geo, block_table, table_width, writes);
    else if (dtype == TS_BF16)
        latent_prepare_kernel<__nv_bfloat16><<<num_tokens, 128, 0, stream>>>((const __nv_bfloat16*)y, y_stride, q_rank, rank,
            rot, wq, wkv, eps, freq, positions, seq_of_token, (__nv_bfloat16*)cq, (__nv_bfloat16*)k_pool, geo, block_table,
            table_width, writes);
    else
        return ts_fail("latent_prepare: unknown dtype code %d", dtype);
    TS_LAUNCH_CHECK("latent_prepare");
    return 0;
}

template <typename T, int MAXR>
__global__ void __launch_bounds__(LA_WARPS * 32)
latent_attention_kernel(const float* __restrict__ q_lat, long long ql_token_stride, long long ql_head_stride,
                        const T* __restrict__ q, long long q_stride, int q_head_width, int q_rot_offset,
                        const float* __restrict__ freq, const T* __restrict__ k_pool, KVGeometry geo,
                        const int* __restrict__ block_table, int table_width, const int* __restrict__ positions,
                        const int* __restrict__ seq_of_token, T* __restrict__ out, int heads, int rank, int rot, float scale,
                        int window, int split_keys, float* __restrict__ partial) {
    extern __shared__ float smem[];
    const int width = rank + rot, pitch = width + 1;
    float* keys = smem;                                   // [LA_KEYS][pitch]
    float* qs = keys + LA_KEYS * pitch;                   // [LA_WARPS][width]
    const int t = blockIdx.x;
    const int seq = seq_of_token[t];
    if (seq < 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y * LA_WARPS + warp;
    const bool head = h < heads;
    const int pos = positions[t];
    float* mine = qs + warp * width;
    if (head) {
        const float* ql = q_lat + (long long)t * ql_token_stride + (long long)h * ql_head_stride;
        for (int d = lane; d < rank; d += 32) mine[d] = ql[d];
        const T* qr = q + (long long)t * q_stride + (long long)h * q_head_width + q_rot_offset;
        const int half = rot / 2;
        for (int i = lane; i < half; i += 32) {
            float sn, cs;
            sincosf((float)pos * freq[i], &sn, &cs);
            const float u = to_float<T>(qr[i]), v = to_float<T>(qr[i + half]);
            mine[rank + i] = u * cs - v * sn;
            mine[rank + i + half] = v * cs + u * sn;
        }
    }
    float o[MAXR];
#pragma unroll
    for (int m = 0; m < MAXR; ++m) o[m] = 0.f;
    float mx = -INFINITY, l = 0.f;
    const int first_key = window > 0 ? max(0, pos - window + 1) : 0;
    // with `split_keys`, CTA z of a token takes keys [first + z * split, first + (z + 1) * split) and leaves a partial result
    const int lo = first_key + (split_keys > 0 ? (int)blockIdx.z * split_keys : 0);
    const int hi = split_keys > 0 ? min(pos, lo + split_keys - 1) : pos;
    const int* table = block_table + (long long)seq * table_width;
    constexpr int VN = 16 / sizeof(T);
    const bool vector = width % VN == 0 && ((geo.page_stride | geo.entry_offset) % VN) == 0 &&
                        (reinterpret_cast<uintptr_t>(k_pool) & 15) == 0;
    const int chunks = width / VN;
    for (int j0 = lo; j0 <= hi; j0 += LA_KEYS) {
        __syncthreads();                                  // the tile before has been read (and, first, qs written)
        const int n = min(LA_KEYS, hi - j0 + 1);
        if (vector) {                                     // a warp a key row at a time, 16 bytes a lane
            for (int jj = warp; jj < n; jj += LA_WARPS) {
                const int j = j0 + jj;
                const int page = table[j / geo.page_tokens];
                const bool in = page >= 0 && page < geo.num_pages;
                const T* src = k_pool + (long long)(in ? page : 0) * geo.page_stride + geo.entry_offset +
                               (long long)(j % geo.page_tokens) * width;
                for (int c = lane; c < chunks; c += 32) {
                    uint4 v = make_uint4(0, 0, 0, 0);
                    if (in) v = *reinterpret_cast<const uint4*>(src + c * VN);
                    const T* el = reinterpret_cast<const T*>(&v);
#pragma unroll
                    for (int i = 0; i < VN; ++i) keys[jj * pitch + c * VN + i] = to_float<T>(el[i]);
                }
            }
        } else {
            for (int e = threadIdx.x; e < n * width; e += blockDim.x) {
                const int jj = e / width, d = e % width;
                const int j = j0 + jj;
                const int page = table[j / geo.page_tokens];
                float x = 0.f;
                if (page >= 0 && page < geo.num_pages)
                    x = to_float<T>(k_pool[(long long)page * geo.page_stride + geo.entry_offset +
                                           (long long)(j % geo.page_tokens) * width + d]);
                keys[jj * pitch + d] = x;
            }
        }
        __syncthreads();
        if (!head) continue;
        float s = -INFINITY;
        if (lane < n) {
            const float* kr = keys + lane * pitch;
            float acc = 0.f;
            for (int d = 0; d < width; ++d) acc = fmaf(mine[d], kr[d], acc);
            s = acc * scale;
        }
        const float m_new = fmaxf(mx, warp_max(s));
        const float corr = expf(mx - m_new);              // 0 at the first tile (mx = -inf)
        const float pr = lane < n ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(pr);
        mx = m_new;
#pragma unroll
        for (int m = 0; m < MAXR; ++m) o[m] *= corr;
        for (int jj = 0; jj < n; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, pr, jj);
            const float* kr = keys + jj * pitch;
#pragma unroll
            for (int m = 0; m < MAXR; ++m) {
                const int d = lane + 32 * m;
                if (d < rank) o[m] = fmaf(pj, kr[d], o[m]);
            }
        }
    }
    if (!head) return;
    if (split_keys > 0) {                                 // [token, head, split]: maximum, sum, then the unscaled output
        float* dst = partial + (((long long)t * heads + h) * gridDim.z + blockIdx.z) * (rank + 2);
        if (lane == 0) { dst[0] = mx; dst[1] = l; }
#pragma unroll
        for (int m = 0; m < MAXR; ++m) {
            const int d = lane + 32 * m;
            if (d < rank) dst[2 + d] = o[m];
        }
        return;
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    T* dst = out + ((long long)t * heads + h) * rank;
#pragma unroll
    for (int m = 0; m < MAXR; ++m) {
        const int d = lane + 32 * m;
        if (d < rank) dst[d] = from_float<T>(o[m] * inv);
    }
}

// Splits of one (token, head) merged in the order of the keys: a split that held no key has sum 0 and counts for nothing.
// One CTA an item: the first warp turns the splits' maxima and sums into one weight a split, then every thread adds up
// its channels over the splits.
constexpr int LC_MAX_SPLITS = 1024;

template <typename T>
__global__ void __launch_bounds__(128)
latent_combine_kernel(const float* __restrict__ partial, T* __restrict__ out, long long items, int splits, int rank) {
    __shared__ float weight[LC_MAX_SPLITS];
    const long long item = blockIdx.x;
    const float* p = partial + item * splits * (rank + 2);
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        float mx = -INFINITY;
        for (int z = lane; z < splits; z += 32)
            if (p[(long long)z * (rank + 2) + 1] > 0.f) mx = fmaxf(mx, p[(long long)z * (rank + 2)]);
        mx = warp_max(mx);
        float total = 0.f;
        for (int z = lane; z < splits; z += 32) {
            const float l = p[(long long)z * (rank + 2) + 1];
            const float w = l > 0.f ? expf(p[(long long)z * (rank + 2)] - mx) : 0.f;
            weight[z] = w;
            total += l * w;
        }
        total = warp_sum(total);
        const float inv = total > 0.f ? 1.f / total : 0.f;
        for (int z = lane; z < splits; z += 32) weight[z] *= inv;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < rank; d += blockDim.x) {
        float acc = 0.f;
        for (int z = 0; z < splits; ++z) acc = fmaf(p[(long long)z * (rank + 2) + 2 + d], weight[z], acc);
        out[item * rank + d] = from_float<T>(acc);
    }
}

template <typename T>
static int launch_latent(const float* q_lat, long long ql_t, long long ql_h, const void* q, long long q_stride,
                         int q_head_width, int q_rot_offset, const float* freq, const void* k_pool, KVGeometry geo,
                         const int* block_table, int table_width, const int* positions, const int* seq_of_token, void* out,
                         int num_tokens, int heads, int rank, int rot, float scale, int window, int split_keys, int splits,
                         float* partial, cudaStream_t stream) {
    const int width = rank + rot;
    const size_t smem = (size_t)(LA_KEYS * (width + 1) + LA_WARPS * width) * sizeof(float);
    dim3 grid(num_tokens, (heads + LA_WARPS - 1) / LA_WARPS, split_keys > 0 ? splits : 1);
#define TS_LATENT(MAXR)                                                                                              \
    do {                                                                                                             \
        if (smem > 48 * 1024)                                                                                        \
            cudaFuncSetAttribute(latent_attention_kernel<T, MAXR>, cudaFuncAttributeMaxDynamicSharedMemorySize,      \
                                 (int)smem);                                                                         \
        latent_attention_kernel<T, MAXR><<<grid, LA_WARPS * 32, smem, stream>>>(                                     \
            q_lat, ql_t, ql_h, (const T*)q, q_stride, q_head_width, q_rot_offset, freq, (const T*)k_pool, geo,       \
            block_table, table_width, positions, seq_of_token, (T*)out, heads, rank, rot, scale, window, split_keys, \
            partial);                                                                                                \
    } while (0)
    if (rank <= 128) TS_LATENT(4);
    else if (rank <= 256) TS_LATENT(8);
    else TS_LATENT(16);
#undef TS_LATENT
    TS_LAUNCH_CHECK("latent_attention");
    if (split_keys > 0) {
        const long long items = (long long)num_tokens * heads;
        latent_combine_kernel<T><<<(unsigned)items, 128, 0, stream>>>(partial, (T*)out, items, splits, rank);
        TS_LAUNCH_CHECK("latent_attention (combine)");
    }
    return 0;
}

// How many floats of scratch a call with these sizes needs (0: the step is large enough to run without splits).
TS_API long long ts_latent_attention_scratch_floats(int num_tokens, int heads, int rank, int max_keys) {
    const int groups = (heads + LA_WARPS - 1) / LA_WARPS;
    if ((long long)num_tokens * groups >= 148 || max_keys <= 2 * LA_SPLIT) return 0;
    const int splits = (max_keys + LA_SPLIT - 1) / LA_SPLIT;
    return (long long)num_tokens * heads * splits * (rank + 2);
}

TS_API int ts_latent_attention(const float* q_lat, long long ql_token_stride, long long ql_head_stride, const void* q,
                               long long q_stride, int q_head_width, int q_rot_offset, const float* freq,
                               const void* k_pool, long long page_stride, long long entry_offset, int page_tokens,
                               int num_pages, const int* block_table, int table_width, const int* positions,
                               const int* seq_of_token, void* out, int num_tokens, int heads, int rank, int rot,
                               float scale, int window, int max_keys, float* scratch, long long scratch_floats, int dtype,
                               cudaStream_t stream) {
    TS_REQUIRE(num_tokens >= 0 && heads > 0 && rank > 0 && rot >= 0 && rot % 2 == 0, "latent_attention: bad sizes");
    TS_REQUIRE(rank <= 512, "latent_attention: a latent of %d channels is not supported (up to 512)", rank);
    TS_REQUIRE(rank + rot <= 1024, "latent_attention: cache rows of %d channels are not supported", rank + rot);
    TS_REQUIRE(page_tokens > 0 && table_width > 0 && window >= 0, "latent_attention: bad page geometry");
    TS_REQUIRE(num_tokens <= 2147483647 && heads <= 65535 * LA_WARPS, "latent_attention: grid too large");
    if (num_tokens == 0) return 0;
    KVGeometry geo{page_stride, entry_offset, page_tokens, num_pages};
    // a step of few tokens (decoding) spreads each token's keys over several CTAs, LA_SPLIT keys each, counted from the
    // window's first key; `max_keys` bounds the keys any token of the step sees
    const long long need = ts_latent_attention_scratch_floats(num_tokens, heads, rank, max_keys);
    int split_keys = 0, splits = 1;
    if (need > 0) {
        TS_REQUIRE(scratch != nullptr && scratch_floats >= need, "latent_attention: %lld floats of scratch needed, %lld given",
                   need, scratch_floats);
        split_keys = LA_SPLIT;
        splits = (max_keys + LA_SPLIT - 1) / LA_SPLIT;
        TS_REQUIRE(splits <= LC_MAX_SPLITS, "latent_attention: %d keys need more than %d splits", max_keys, LC_MAX_SPLITS);
    }
    if (dtype == TS_BF16 && ts_latent_mma_supported(rank, rot) && page_stride % 8 == 0 && entry_offset % 8 == 0 &&
        (uintptr_t)k_pool % 16 == 0) {
        // bfloat16 with sizes the tensor-core kernel takes: heads as the rows of mma.sync products
        if (ts_latent_attention_mma_launch(q_lat, ql_token_stride, ql_head_stride, q, q_stride, q_head_width, q_rot_offset,
                                           freq, k_pool, geo, block_table, table_width, positions, seq_of_token, out,
                                           num_tokens, heads, rank, rot, scale, window, split_keys, splits, scratch, stream))
            return 1;
        if (split_keys > 0) {
            const long long items = (long long)num_tokens * heads;
            latent_combine_kernel<__nv_bfloat16><<<(unsigned)items, 128, 0, stream>>>(
                scratch, (__nv_bfloat16*)out, items, splits, rank);
            TS_LAUNCH_CHECK("latent_attention (combine)");
        }
        return 0;
    }
    if (dtype == TS_F32)
        return launch_latent<float>(q_lat, ql_token_stride, ql_head_stride, q, q_stride, q_head_width, q_rot_offset, freq,
                                    k_pool, geo, block_table, table_width, positions, seq_of_token, out, num_tokens, heads,
                                    rank, rot, scale, window, split_keys, splits, scratch, stream);
    if (dtype == TS_BF16)
        return launch_latent<__nv_bfloat16>(q_lat, ql_token_stride, ql_head_stride, q, q_stride, q_head_width, q_rot_offset,
                                            freq, k_pool, geo, block_table, table_width, positions, seq_of_token, out,
                                            num_tokens, heads, rank, rot, scale, window, split_keys, splits, scratch, stream);
    return ts_fail("latent_attention: unknown dtype code %d", dtype);
}
