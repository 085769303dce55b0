// Element-wise gated recurrence whose gates read the current token only (a minGRU):
//
//   z_t = sigmoid(a_t + b_z)        a, u: the projections' outputs for token t (columns of one row of y)
//   c_t = u_t + b_x + 1/2  where u_t + b_x >= 0,  sigmoid(u_t + b_x)  below
//   S_t = (1 - z_t) S_(t-1) + z_t c_t               one number a channel, float32, carried in the request's slot
//   out_t = S_t * silu(g_t)                          g: a third stretch of y's row
//
// Everything after the projections is float32; `out` has the activation dtype.  A request's tokens of
// this step are the rows cu_q[s] .. cu_q[s + 1]; its state is read from and written back to row
// state_slots[s] of `state` (a negative slot: a padding request, nothing is read or written).
//
// Two kernels.  `mingru_scan_kernel`: a thread a (request, channel) walks the request's tokens in order,
// loads a few tokens ahead.  `mingru_scan_chunked_kernel` (steps with long portions): a CTA is a request
// and 32 channels, a lane a channel; every warp takes a stretch of the request's tokens, first reduces it
// to the pair (A, B) with S_end = A S_begin + B, the warps' pairs are chained in order through shared
// memory, then every warp walks its stretch again from its true starting state and writes the outputs.
// Both give each token one fixed order of operations for a given cut of the step into warps' stretches;
// between the two kernels, and between cuts, results differ by rounding only.
#include "common.cuh"

struct MinGRUArgs {
    const void* y; long long y_stride; int z_off, x_off, g_off;     // columns of the three stretches inside a row of y
    const float* z_bias; const float* x_bias;                       // null: no bias
    const int* cu_q; const int* state_slots; int num_seqs;
    float* state; long long state_stride;                           // floats between slots
    void* out; int width;
};

// FAST (outputs of 16 bits): the exponential and the division by their one-instruction forms, whose error of a
// few units in the last place of a float is far below the output's rounding; float32 outputs keep the exact ones.
template <bool FAST>
__device__ __forceinline__ float mingru_sigmoid(float x) {
    return FAST ? __fdividef(1.f, 1.f + __expf(-x)) : 1.f / (1.f + expf(-x));
}

template <bool FAST>
__device__ __forceinline__ void mingru_gates(float a, float u, float bz, float bx, float& z, float& c) {
    z = mingru_sigmoid<FAST>(a + bz);
    const float v = u + bx;
    c = v >= 0.f ? v + 0.5f : mingru_sigmoid<FAST>(v);
}

constexpr int MG_AHEAD = 4;

template <typename TY, typename T>
__global__ void __launch_bounds__(128) mingru_scan_kernel(MinGRUArgs p) {
    constexpr bool FAST = sizeof(T) == 2;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int s = blockIdx.y;
    if (c >= p.width) return;
    const int slot = p.state_slots[s];
    const int t0 = p.cu_q[s], t1 = p.cu_q[s + 1];
    if (slot < 0 || t1 <= t0) return;
    const float bz = p.z_bias ? p.z_bias[c] : 0.f, bx = p.x_bias ? p.x_bias[c] : 0.f;
    float* sp = p.state + (long long)slot * p.state_stride + c;
    float S = *sp;
    const TY* y = (const TY*)p.y;
    T* out = (T*)p.out;
    float a[MG_AHEAD], u[MG_AHEAD], g[MG_AHEAD];
#pragma unroll
    for (int i = 0; i < MG_AHEAD; ++i) {
        const long long row = (long long)min(t0 + i, t1 - 1) * p.y_stride + c;
        a[i] = to_float<TY>(y[row + p.z_off]); u[i] = to_float<TY>(y[row + p.x_off]); g[i] = to_float<TY>(y[row + p.g_off]);
    }
    for (int t = t0; t < t1; t += MG_AHEAD) {
        float an[MG_AHEAD], un[MG_AHEAD], gn[MG_AHEAD];
#pragma unroll
        for (int i = 0; i < MG_AHEAD; ++i) {                 // the next group's loads are under way during this group's chain
            const long long row = (long long)min(t + MG_AHEAD + i, t1 - 1) * p.y_stride + c;
            an[i] = to_float<TY>(y[row + p.z_off]); un[i] = to_float<TY>(y[row + p.x_off]); gn[i] = to_float<TY>(y[row + p.g_off]);
        }
#pragma unroll
        for (int i = 0; i < MG_AHEAD; ++i) {
            if (t + i < t1) {
                float z, cand;
                mingru_gates<FAST>(a[i], u[i], bz, bx, z, cand);
                S = (1.f - z) * S + z * cand;
                out[(long long)(t + i) * p.width + c] = from_float<T>(S * (g[i] * mingru_sigmoid<FAST>(g[i])));
            }
        }
#pragma unroll
        for (int i = 0; i < MG_AHEAD; ++i) { a[i] = an[i]; u[i] = un[i]; g[i] = gn[i]; }
    }
    *sp = S;
}

constexpr int MG_WARPS = 32;
constexpr int MG_BATCH = 8;              // tokens whose loads are under way together

template <typename TY, typename T>
__global__ void __launch_bounds__(MG_WARPS * 32) mingru_scan_chunked_kernel(MinGRUArgs p) {
    constexpr bool FAST = sizeof(T) == 2;
    __shared__ float As[MG_WARPS][32], Bs[MG_WARPS][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + lane;
    const int s = blockIdx.y;
    const int slot = p.state_slots[s];
    const int t0 = p.cu_q[s], t1 = p.cu_q[s + 1];
    if (slot < 0 || t1 <= t0) return;                        // the same for the whole CTA
    const bool live = c < p.width;
    const int cc = live ? c : p.width - 1;
    const int n = t1 - t0, per = (n + MG_WARPS - 1) / MG_WARPS;
    const int w0 = min(t0 + warp * per, t1), w1 = min(w0 + per, t1);
    const float bz = p.z_bias ? p.z_bias[cc] : 0.f, bx = p.x_bias ? p.x_bias[cc] : 0.f;
    const TY* y = (const TY*)p.y;
    // first walk: the stretch as one step S_end = A S_begin + B
    float A = 1.f, B = 0.f;
    for (int t = w0; t < w1; t += MG_BATCH) {
        float a[MG_BATCH], u[MG_BATCH];
#pragma unroll
        for (int i = 0; i < MG_BATCH; ++i) {                 // rows beyond the stretch: its last row again, not used
            const long long row = (long long)min(t + i, w1 - 1) * p.y_stride + cc;
            a[i] = to_float<TY>(y[row + p.z_off]); u[i] = to_float<TY>(y[row + p.x_off]);
        }
#pragma unroll
        for (int i = 0; i < MG_BATCH; ++i) {
            if (t + i < w1) {
                float z, cand;
                mingru_gates<FAST>(a[i], u[i], bz, bx, z, cand);
                A *= 1.f - z;
                B = (1.f - z) * B + z * cand;
            }
        }
    }
    As[warp][lane] = A;
    Bs[warp][lane] = B;
    __syncthreads();
    float* sp = p.state + (long long)slot * p.state_stride + cc;
    float S = *sp;
    for (int w = 0; w < warp; ++w) S = As[w][lane] * S + Bs[w][lane];      // the state this warp's stretch starts from
    T* out = (T*)p.out;
    for (int t = w0; t < w1; t += MG_BATCH) {
        float a[MG_BATCH], u[MG_BATCH], g[MG_BATCH];
#pragma unroll
        for (int i = 0; i < MG_BATCH; ++i) {
            const long long row = (long long)min(t + i, w1 - 1) * p.y_stride + cc;
            a[i] = to_float<TY>(y[row + p.z_off]); u[i] = to_float<TY>(y[row + p.x_off]); g[i] = to_float<TY>(y[row + p.g_off]);
        }
#pragma unroll
        for (int i = 0; i < MG_BATCH; ++i) {
            if (t + i < w1) {
                float z, cand;
                mingru_gates<FAST>(a[i], u[i], bz, bx, z, cand);
                S = (1.f - z) * S + z * cand;
                if (live) out[(long long)(t + i) * p.width + c] = from_float<T>(S * (g[i] * mingru_sigmoid<FAST>(g[i])));
            }
        }
    }
    if (live && warp == MG_WARPS - 1) *sp = S;               // the last warp ends at the request's last token (or holds the state unchanged)
}

// y: float32 (y_dtype TS_F32) or the activation dtype; out: the activation dtype `dtype`.  `max_q_len`: the most
// tokens a request feeds in this step (chooses the kernel; 0: unknown, the walk in order).
TS_API int ts_mingru_scan(const void* y, long long y_stride, int z_off, int x_off, int g_off, int y_dtype,
                          const float* z_bias, const float* x_bias, const int* cu_q, const int* state_slots, int num_seqs,
                          float* state, long long state_stride, void* out, int width, int num_tokens, int max_q_len,
                          int dtype, cudaStream_t stream) {
    TS_REQUIRE(width > 0 && num_seqs >= 0 && num_tokens >= 0, "mingru_scan: bad sizes");
    TS_REQUIRE(state != nullptr && state_stride >= width, "mingru_scan: the state slot holds fewer than %d floats", width);
    TS_REQUIRE(y_dtype == TS_F32 || y_dtype == dtype, "mingru_scan: the projections are float32 or of the activation dtype");
    if (num_seqs == 0 || num_tokens == 0) return 0;
    MinGRUArgs p{y, y_stride, z_off, x_off, g_off, z_bias, x_bias, cu_q, state_slots, num_seqs, state, state_stride, out, width};
    const bool chunked = max_q_len >= 4 * MG_WARPS;
    const dim3 grid(chunked ? (width + 31) / 32 : (width + 127) / 128, num_seqs);
    const int threads = chunked ? MG_WARPS * 32 : 128;
#define TS_MINGRU(TY, T)                                                                   \
    do {                                                                                   \
        if (chunked) mingru_scan_chunked_kernel<TY, T><<<grid, threads, 0, stream>>>(p);   \
        else mingru_scan_kernel<TY, T><<<grid, threads, 0, stream>>>(p);                   \
    } while (0)
    if (dtype == TS_F32) TS_MINGRU(float, float);
    else if (dtype == TS_BF16 && y_dtype == TS_F32) TS_MINGRU(float, __nv_bfloat16);
    else if (dtype == TS_BF16) TS_MINGRU(__nv_bfloat16, __nv_bfloat16);
    else return ts_fail("mingru_scan: unknown dtype code %d", dtype);
#undef TS_MINGRU
    TS_LAUNCH_CHECK("mingru_scan");
    return 0;
}
