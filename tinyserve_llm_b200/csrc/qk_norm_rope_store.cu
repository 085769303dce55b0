// What lies between the q/k/v projection and the attention of a mixer whose queries and keys are
// normed over the whole projection:
//
//   q = y_q + b_q,  k = y_k + b_k,  v = y_v + b_v                      (biases optional)
//   q = q / sqrt(mean(q^2) + eps) * w_q     over all heads' channels at once, likewise k   (optional);
//       with `norm_per_head` every head is normed by itself and w_q, w_k hold one head's channels
//   q = q * (1 + temp_coef * ln(floor((position + 1) / temp_every) + 1))             (temp_every > 0)
//   rotate-half rotation of the first `rot` channels of every head of q and k: channel i pairs with
//   i + rot/2, angle = position * freq[i], cos and sin both multiplied by `magnitude`
//   k and v go to the token's slot of the paged cache, q to a compact [tokens, heads * dim] tensor.
//
// Keys and values may differ in their head size and in their number of heads (`v_heads`: several key heads over
// one value head), so the value pool has a geometry of its own.
// One CTA a token; sums, angles and the rotation are float32, the stores round to the activation dtype.
#include "common.cuh"

struct QKPrepareArgs {
    const void* y; long long y_stride; int q_off, k_off, v_off;     // columns of q, k and v inside a row of y
    const float* q_bias; const float* k_bias; const float* v_bias;
    const float* q_weight; const float* k_weight; float eps;        // null weights: no norm
    const float* freq; int rot; float magnitude;
    const int* positions; const int* seq_of_token;
    void* q_out;
    void* k_pool; void* v_pool; KVGeometry k_geo; KVGeometry v_geo;
    const int* block_table; int table_width; int writes;
    int heads, kv_heads, dim, vdim, v_heads;
    int norm_per_head; float temp_coef; int temp_every;
};

template <typename T>
__global__ void qk_norm_rope_store_kernel(QKPrepareArgs p) {
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const int seq = p.seq_of_token[t];
    const int nq = p.heads * p.dim, nk = p.kv_heads * p.dim, nv = p.v_heads * p.vdim;
    T* q_out = (T*)p.q_out + (long long)t * nq;
    if (seq < 0) {                                    // a padding row
        for (int e = threadIdx.x; e < nq; e += blockDim.x) q_out[e] = from_float<T>(0.f);
        return;
    }
    const T* row = (const T*)p.y + (long long)t * p.y_stride;
    const T* yq = row + p.q_off;
    const T* yk = row + p.k_off;
    const T* yv = row + p.v_off;
    // what does not depend on the sums is asked for first: the position and the page
    const int pos = p.positions[t];
    const int half = p.rot / 2;
    const int page = p.writes ? p.block_table[(long long)seq * p.table_width + pos / p.k_geo.page_tokens] : -1;
    float inv_q = 1.f, inv_k = 1.f;
    extern __shared__ float inv_heads[];              // norm_per_head: 1 / rms of every q head, then of every k head
    if (p.norm_per_head && (p.q_weight || p.k_weight)) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
        for (int hh = warp; hh < p.heads + p.kv_heads; hh += nwarps) {      // a warp a head
            const bool is_q = hh < p.heads;
            const int e0 = (is_q ? hh : hh - p.heads) * p.dim;
            const T* y = is_q ? yq : yk;
            const float* bias = is_q ? p.q_bias : p.k_bias;
            float acc = 0.f;
            if (is_q ? p.q_weight != nullptr : p.k_weight != nullptr)
                for (int i = lane; i < p.dim; i += 32) {
                    const float x = to_float<T>(y[e0 + i]) + (bias ? bias[e0 + i] : 0.f);
                    acc += x * x;
                }
            acc = warp_sum(acc);
            if (lane == 0) inv_heads[hh] = 1.f / sqrtf(acc / (float)p.dim + p.eps);
        }
        __syncthreads();
    } else if (p.q_weight || p.k_weight) {            // both sums in one pass over the row, then two reductions
        float acc_q = 0.f, acc_k = 0.f;
        if (p.q_weight)
            for (int e = threadIdx.x; e < nq; e += blockDim.x) {
                const float x = to_float<T>(yq[e]) + (p.q_bias ? p.q_bias[e] : 0.f);
                acc_q += x * x;
            }
        if (p.k_weight)
            for (int e = threadIdx.x; e < nk; e += blockDim.x) {
                const float x = to_float<T>(yk[e]) + (p.k_bias ? p.k_bias[e] : 0.f);
                acc_k += x * x;
            }
        if (p.q_weight) {
            inv_q = 1.f / sqrtf(block_sum(acc_q, scratch) / (float)nq + p.eps);
            __syncthreads();
        }
        if (p.k_weight) inv_k = 1.f / sqrtf(block_sum(acc_k, scratch) / (float)nk + p.eps);
    }
    // `heads_at`: where this projection's heads start in inv_heads; `gain` multiplies every element (the query's temperature)
    auto element = [&](const T* y, const float* bias, const float* weight, float inv, int heads_at, float gain, int e) {
        const float x = to_float<T>(y[e]) + (bias ? bias[e] : 0.f);
        if (!weight) return x * gain;
        if (p.norm_per_head) return x * inv_heads[heads_at + e / p.dim] * weight[e % p.dim] * gain;
        return x * inv * weight[e] * gain;
    };
    const float temperature = p.temp_every > 0
        ? 1.f + p.temp_coef * logf((float)((pos + 1) / p.temp_every) + 1.f) : 1.f;
    // One thread a rotated pair (i, i + rot/2): one sincosf for both; channels past `rot` pass unchanged.
    auto rotate_into = [&](const T* y, const float* bias, const float* weight, float inv, int heads_at, float gain, int n,
                           auto&& store) {
        for (int e = threadIdx.x; e < n; e += blockDim.x) {
            const int i = e % p.dim;
            if (p.freq && i < p.rot) {
                if (i >= half) continue;                   // written by the pair's first channel
                const float u = element(y, bias, weight, inv, heads_at, gain, e);
                const float v = element(y, bias, weight, inv, heads_at, gain, e + half);
                float sn, cs;
                sincosf((float)pos * p.freq[i], &sn, &cs);
                sn *= p.magnitude;
                cs *= p.magnitude;
                store(e, u * cs - v * sn);
                store(e + half, v * cs + u * sn);
            } else {
                store(e, element(y, bias, weight, inv, heads_at, gain, e));
            }
        }
    };
    rotate_into(yq, p.q_bias, p.q_weight, inv_q, 0, temperature, nq, [&](int e, float x) { q_out[e] = from_float<T>(x); });
    if (!p.writes || page < 0 || page >= p.k_geo.num_pages) return;
    const int slot = pos % p.k_geo.page_tokens;
    T* kp = (T*)p.k_pool + (long long)page * p.k_geo.page_stride + p.k_geo.entry_offset;
    T* vp = (T*)p.v_pool + (long long)page * p.v_geo.page_stride + p.v_geo.entry_offset;
    rotate_into(yk, p.k_bias, p.k_weight, inv_k, p.heads, 1.f, nk, [&](int e, float x) {
        const int h = e / p.dim, i = e % p.dim;
        kp[((long long)h * p.k_geo.page_tokens + slot) * p.dim + i] = from_float<T>(x);
    });
    for (int e = threadIdx.x; e < nv; e += blockDim.x) {
        const int h = e / p.vdim, i = e % p.vdim;
        vp[((long long)h * p.v_geo.page_tokens + slot) * p.vdim + i] =
            from_float<T>(to_float<T>(yv[e]) + (p.v_bias ? p.v_bias[e] : 0.f));
    }
}

TS_API int ts_qk_norm_rope_store(const void* y, long long y_stride, int q_off, int k_off, int v_off, const float* q_bias,
                                 const float* k_bias, const float* v_bias, const float* q_weight, const float* k_weight,
                                 float eps, const float* freq, int rot, float magnitude, const int* positions,
                                 const int* seq_of_token, void* q_out, void* k_pool, void* v_pool, long long k_page_stride,
                                 long long k_entry_offset, long long v_page_stride, long long v_entry_offset,
                                 int page_tokens, int num_pages, const int* block_table, int table_width, int writes,
                                 int num_tokens, int heads, int kv_heads, int dim, int vdim, int dtype,
                                 int norm_per_head, float temp_coef, int temp_every, int value_heads, cudaStream_t stream) {
    TS_REQUIRE(value_heads >= 0, "qk_norm_rope_store: bad number of value heads");
    TS_REQUIRE(heads > 0 && kv_heads > 0 && dim > 0 && vdim > 0 && num_tokens >= 0, "qk_norm_rope_store: bad sizes");
    TS_REQUIRE(rot >= 0 && rot <= dim && rot % 2 == 0, "qk_norm_rope_store: rotation over %d of %d channels", rot, dim);
    TS_REQUIRE(page_tokens > 0 && table_width > 0, "qk_norm_rope_store: bad page geometry");
    if (num_tokens == 0) return 0;
    QKPrepareArgs p{y, y_stride, q_off, k_off, v_off, q_bias, k_bias, v_bias, q_weight, k_weight, eps,
                    rot > 0 ? freq : nullptr, rot, magnitude, positions, seq_of_token, q_out, k_pool, v_pool,
                    KVGeometry{k_page_stride, k_entry_offset, page_tokens, num_pages},
                    KVGeometry{v_page_stride, v_entry_offset, page_tokens, num_pages}, block_table, table_width, writes,
                    heads, kv_heads, dim, vdim, value_heads > 0 ? value_heads : kv_heads, norm_per_head, temp_coef, temp_every};
    const size_t smem = norm_per_head ? (size_t)(heads + kv_heads) * sizeof(float) : 0;
    TS_REQUIRE(smem <= 32 * 1024, "qk_norm_rope_store: %d heads are not supported", heads + kv_heads);
    // many tokens: small CTAs, many of them on an SM (a CTA's life is a chain of loads and two sums); few tokens: wide ones
    const int threads = num_tokens >= 512 ? 128 : (heads * dim >= 2048 ? 512 : 256);
    if (dtype == TS_F32) qk_norm_rope_store_kernel<float><<<num_tokens, threads, smem, stream>>>(p);
    else if (dtype == TS_BF16) qk_norm_rope_store_kernel<__nv_bfloat16><<<num_tokens, threads, smem, stream>>>(p);
    else return ts_fail("qk_norm_rope_store: unknown dtype code %d", dtype);
    TS_LAUNCH_CHECK("qk_norm_rope_store");
    return 0;
}

// out[t, c] = a[t, c] * sigmoid(gate[t, c]) * scale, each operand with a row stride of its own (the
// result may be a column stretch of a wider tensor).  An output gate on concatenated heads.
template <typename T>
__global__ void sigmoid_gate_kernel(const T* __restrict__ a, long long a_stride, const T* __restrict__ gate,
                                    long long gate_stride, T* __restrict__ out, long long out_stride, long long total,
                                    int cols, float scale) {
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long t = idx / cols;
        const int c = (int)(idx % cols);
        const float g = to_float<T>(gate[t * gate_stride + c]);
        out[t * out_stride + c] = from_float<T>(to_float<T>(a[t * a_stride + c]) / (1.f + expf(-g)) * scale);
    }
}

TS_API int ts_sigmoid_gate(const void* a, long long a_stride, const void* gate, long long gate_stride, void* out,
                           long long out_stride, int num_tokens, int cols, float scale, int dtype, cudaStream_t stream) {
    TS_REQUIRE(num_tokens >= 0 && cols > 0, "sigmoid_gate: bad sizes");
    if (num_tokens == 0) return 0;
    const long long total = (long long)num_tokens * cols;
    const unsigned blocks = (unsigned)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    if (dtype == TS_F32)
        sigmoid_gate_kernel<float><<<blocks, 256, 0, stream>>>((const float*)a, a_stride, (const float*)gate, gate_stride,
                                                               (float*)out, out_stride, total, cols, scale);
    else if (dtype == TS_BF16)
        sigmoid_gate_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)a, a_stride,
            (const __nv_bfloat16*)gate, gate_stride, (__nv_bfloat16*)out, out_stride, total, cols, scale);
    else
        return ts_fail("sigmoid_gate: unknown dtype code %d", dtype);
    TS_LAUNCH_CHECK("sigmoid_gate");
    return 0;
}
