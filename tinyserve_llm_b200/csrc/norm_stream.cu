// RMS norms around a residual stream that is kept in float32 whatever the activation dtype.
//
// One kernel does what lies between two sublayers of a block that norms each sublayer's input and
// output:  s = stream + closing(branch),  stream' = s,  out = opening(s)  with
//   closing(b) = b / sqrt(mean(b^2) + eps) * w_close      (the norm after the sublayer that made b)
//   opening(s) = s / sqrt(mean(s^2) + eps) * w_open       (the norm before the next sublayer)
// Every part is optional: no branch (the stream is only normed: a block's first norm after a block
// that closed its own branch), no opening weight (the branch is only added), `rows` (only these
// rows are normed into a compact output and the stream is not written: the final norm of the
// wanted places), `ids` (the row is table[ids[r]] * scale and starts the stream: the embedding; with
// `pos_freq` a sinusoidal position vector is added to it: entry 2i gets sin(position * pos_freq[i]),
// entry 2i + 1 the cosine of the same angle, the angle a float32 product; with `w_start` the gathered row is
// itself normed with that weight, in the way the opening norm is, before it starts the stream: a norm on the embedding).
// Statistics, weights, the sum and the stream are float32; the branch and `out` have the activation
// dtype.  The weights are given as they multiply (an offset of the stored weight is added by the host).
//
// `flags`: TS_NORM_CENTERED makes the opening norm a layer norm without bias,
//   opening(s) = (s - mean(s)) / sqrt(mean((s - mean(s))^2) + eps) * w_open;
// TS_NORM_PLAIN_ADD adds the branch as it is (a block that norms only the inputs of its sublayers).
#include "common.cuh"

enum { TS_NORM_CENTERED = 1, TS_NORM_PLAIN_ADD = 2 };

template <typename T>
__global__ void stream_norm_kernel(const T* __restrict__ branch, const float* __restrict__ w_close, float* stream,
                                   const float* __restrict__ w_open, T* __restrict__ out,
                                   const int* __restrict__ rows, int width, float eps, const T* __restrict__ table,
                                   const int* __restrict__ ids, int table_rows, float scale, int write_stream,
                                   int flags, const int* __restrict__ positions, const float* __restrict__ pos_freq,
                                   const float* __restrict__ w_start) {
    extern __shared__ float row[];                // width floats, then 32 of scratch
    float* scratch = row + width;
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    if (src < 0) return;                          // a padding row
    float* sr = stream + (long long)src * width;
    if (ids) {
        const int id = ids[src];
        const bool zeros = id < 0 || id >= table_rows;
        const T* tr = table + (long long)(zeros ? 0 : id) * width;
        if (pos_freq) {
            const float pos = (float)positions[src];
            for (int i = threadIdx.x; i < width; i += blockDim.x) {
                const float angle = pos * pos_freq[i >> 1];
                row[i] = (zeros ? 0.f : to_float<T>(tr[i]) * scale) + ((i & 1) ? cosf(angle) : sinf(angle));
            }
        } else {
            for (int i = threadIdx.x; i < width; i += blockDim.x) row[i] = zeros ? 0.f : to_float<T>(tr[i]) * scale;
        }
        if (w_start) {                            // each thread reads back only the elements it wrote
            float mean = 0.f;
            if (flags & TS_NORM_CENTERED) {
                float sum = 0.f;
                for (int i = threadIdx.x; i < width; i += blockDim.x) sum += row[i];
                mean = block_sum(sum, scratch) / (float)width;
                __syncthreads();
            }
            float acc = 0.f;
            for (int i = threadIdx.x; i < width; i += blockDim.x) acc += (row[i] - mean) * (row[i] - mean);
            const float inv = 1.f / sqrtf(block_sum(acc, scratch) / (float)width + eps);
            __syncthreads();                      // scratch is used again below
            for (int i = threadIdx.x; i < width; i += blockDim.x) row[i] = (row[i] - mean) * inv * w_start[i];
        }
    } else if (branch && (flags & TS_NORM_PLAIN_ADD)) {
        const T* br = branch + (long long)src * width;
        for (int i = threadIdx.x; i < width; i += blockDim.x) row[i] = sr[i] + to_float<T>(br[i]);
    } else if (branch) {
        const T* br = branch + (long long)src * width;
        float acc = 0.f;
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            const float b = to_float<T>(br[i]);
            row[i] = b;
            acc += b * b;
        }
        const float inv = 1.f / sqrtf(block_sum(acc, scratch) / (float)width + eps);
        __syncthreads();                          // scratch is used again below
        for (int i = threadIdx.x; i < width; i += blockDim.x) row[i] = sr[i] + row[i] * inv * w_close[i];
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) row[i] = sr[i];
    }
    if (write_stream && (ids || branch))
        for (int i = threadIdx.x; i < width; i += blockDim.x) sr[i] = row[i];
    if (!w_open) return;
    float mean = 0.f;
    if (flags & TS_NORM_CENTERED) {
        float sum = 0.f;
        for (int i = threadIdx.x; i < width; i += blockDim.x) sum += row[i];
        mean = block_sum(sum, scratch) / (float)width;
        __syncthreads();                          // scratch is used again below
    }
    float acc = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) acc += (row[i] - mean) * (row[i] - mean);
    const float inv = 1.f / sqrtf(block_sum(acc, scratch) / (float)width + eps);
    T* o = out + (long long)r * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = from_float<T>((row[i] - mean) * inv * w_open[i]);
}

TS_API int ts_stream_norm(const void* branch, const float* w_close, float* stream, const float* w_open, void* out,
                          const int* rows, int count, int width, float eps, const void* table, const int* ids,
                          int table_rows, float scale, int flags, int dtype, const int* positions, const float* pos_freq,
                          const float* w_start, cudaStream_t stream_handle) {
    TS_REQUIRE(count >= 0 && width > 0, "stream_norm: bad sizes rows=%d width=%d", count, width);
    TS_REQUIRE(stream != nullptr, "stream_norm: no residual stream");
    TS_REQUIRE(!(branch && !w_close && !(flags & TS_NORM_PLAIN_ADD)), "stream_norm: a branch needs the weight of its closing norm");
    TS_REQUIRE(!(w_open && !out), "stream_norm: an opening norm needs an output");
    TS_REQUIRE(!(ids && (!table || branch)), "stream_norm: token ids need the table and exclude a branch");
    TS_REQUIRE(!(pos_freq && (!ids || !positions)), "stream_norm: a position vector needs token ids and positions");
    TS_REQUIRE(!(w_start && !ids), "stream_norm: a norm on the embedding needs token ids");
    TS_REQUIRE(width <= 48 * 1024, "stream_norm: rows of %d elements are not supported", width);
    if (count == 0) return 0;
    // few rows (decoding) are bound by the chain of loads, not by their number: about four elements a thread and pass;
    // many rows keep more CTAs on an SM instead
    const int wide = width >= 4096 ? 1024 : width >= 2048 ? 512 : width >= 1024 ? 256 : 128;
    const int threads = count <= 512 ? wide : (width >= 1024 ? 256 : 128);
    const size_t smem = (size_t)(width + 32) * sizeof(float);
    const int write = rows ? 0 : 1;
#define TS_STREAM_NORM(TYPE)                                                                                      \
    do {                                                                                                          \
        if (smem > 48 * 1024)                                                                                     \
            cudaFuncSetAttribute(stream_norm_kernel<TYPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        stream_norm_kernel<TYPE><<<count, threads, smem, stream_handle>>>(                                        \
            (const TYPE*)branch, w_close, stream, w_open, (TYPE*)out, rows, width, eps, (const TYPE*)table, ids,  \
            table_rows, scale, write, flags, positions, pos_freq, w_start);                                             \
    } while (0)
    if (dtype == TS_F32) TS_STREAM_NORM(float);
    else if (dtype == TS_BF16) TS_STREAM_NORM(__nv_bfloat16);
    else return ts_fail("stream_norm: unknown dtype code %d", dtype);
#undef TS_STREAM_NORM
    TS_LAUNCH_CHECK("stream_norm");
    return 0;
}
