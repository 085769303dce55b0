// Differential attention's last step.  Every head has two score maps over the same values; the attention
// kernels treat the maps as heads of their own and leave, per token, the outputs [group][map][head in group][vdim]
// (a group = the query heads of one key/value head; with this order the heads that share a key head lie side by
// side).  Here, for head h = group * r + i:
//   d = a_1 - lambda * a_2,   o = d / sqrt(mean(d^2) + eps) * out_scale        over the head's vdim channels
// with one lambda for the layer.  The norm has no weight.  The maps come in float32 or in the activation dtype;
// the difference, the mean and the norm are float32; o has the activation dtype, heads in their own order.
//
// Also: the logits' last step of designs that scale and cap them, x <- cap * tanh(x * scale / cap).
#include "common.cuh"

template <typename TIN, typename TOUT>
__global__ void __launch_bounds__(128)
difference_head_norm_kernel(const TIN* __restrict__ maps, long long maps_stride, TOUT* __restrict__ out, long long out_stride,
                            const int* __restrict__ seq_of_token, long long items, int heads, int per_group, int vdim,
                            float lambda, float eps, float out_scale) {
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= items) return;
    const long long t = item / heads;
    const int h = (int)(item % heads);
    if (seq_of_token && seq_of_token[t] < 0) return;          // a padding row
    const int group = h / per_group, i = h % per_group;
    const TIN* a1 = maps + t * maps_stride + ((long long)(group * 2) * per_group + i) * vdim;
    const TIN* a2 = a1 + (long long)per_group * vdim;
    float d[8];                                               // vdim <= 256
    float acc = 0.f;
#pragma unroll
    for (int m = 0; m < 8; ++m) {
        const int c = lane + 32 * m;
        d[m] = c < vdim ? to_float<TIN>(a1[c]) - lambda * to_float<TIN>(a2[c]) : 0.f;
        acc = fmaf(d[m], d[m], acc);
    }
    const float inv = out_scale / sqrtf(warp_sum(acc) / (float)vdim + eps);
    TOUT* o = out + t * out_stride + (long long)h * vdim;
#pragma unroll
    for (int m = 0; m < 8; ++m) {
        const int c = lane + 32 * m;
        if (c < vdim) o[c] = from_float<TOUT>(d[m] * inv);
    }
}

// maps: [tokens, 2 * heads * vdim] (`maps_f32` 1: float32, 0: the activation dtype); out: [tokens, heads * vdim].
TS_API int ts_difference_head_norm(const void* maps, long long maps_stride, int maps_f32, void* out, long long out_stride,
                                   const int* seq_of_token, int num_tokens, int heads, int kv_heads, int vdim, float lambda,
                                   float eps, float out_scale, int dtype, cudaStream_t stream) {
    TS_REQUIRE(num_tokens >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0, "difference_head_norm: bad head counts");
    TS_REQUIRE(vdim > 0 && vdim <= 256, "difference_head_norm: heads of %d value channels are not supported (up to 256)", vdim);
    if (num_tokens == 0) return 0;
    const long long items = (long long)num_tokens * heads;
    const unsigned blocks = (unsigned)((items + 3) / 4);
    const int r = heads / kv_heads;
#define TS_DIFF(TIN, TOUT)                                                                                             \
    difference_head_norm_kernel<TIN, TOUT><<<blocks, 128, 0, stream>>>((const TIN*)maps, maps_stride, (TOUT*)out,      \
        out_stride, seq_of_token, items, heads, r, vdim, lambda, eps, out_scale)
    if (dtype == TS_F32) TS_DIFF(float, float);
    else if (dtype == TS_BF16 && maps_f32) TS_DIFF(float, __nv_bfloat16);
    else if (dtype == TS_BF16) TS_DIFF(__nv_bfloat16, __nv_bfloat16);
    else return ts_fail("difference_head_norm: unknown dtype code %d", dtype);
#undef TS_DIFF
    TS_LAUNCH_CHECK("difference_head_norm");
    return 0;
}

__global__ void scale_tanh_cap_kernel(float* __restrict__ x, long long total, float scale, float cap) {
    const float inv = cap > 0.f ? scale / cap : 0.f;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x)
        x[idx] = cap > 0.f ? cap * tanhf(x[idx] * inv) : x[idx] * scale;
}

// x (float32, in place) <- cap * tanh(x * scale / cap); cap 0: x * scale only.
TS_API int ts_scale_tanh_cap(float* x, long long total, float scale, float cap, cudaStream_t stream) {
    TS_REQUIRE(total >= 0 && cap >= 0.f, "scale_tanh_cap: bad arguments");
    if (total == 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    scale_tanh_cap_kernel<<<blocks, 256, 0, stream>>>(x, total, scale, cap);
    TS_LAUNCH_CHECK("scale_tanh_cap");
    return 0;
}
