// Routed experts: every token goes through its `top` best experts of `experts` small gated
// feed-forward layers, and the outputs are added with the softmax of the chosen logits as weights.
//
//   ts_moe_route     per token: the `top` largest router logits (float32, bias added here; ties go to
//                    the lower index), their softmax, and a count per expert.  `scoring` 1: a chosen
//                    expert's share is sigmoid(logit) instead, not renormalised.  `scoring` 2: scores are the
//                    softmax over ALL router outputs; the choice goes by score + correction[e] among the
//                    outputs of the `keep` best of `groups` equal groups of neighbours (a group ranks by its
//                    largest choice score); a chosen output's share is its score (without the correction)
//                    divided by the chosen scores' sum + share_eps, times weight_scale.  Outputs from
//                    `real_experts` on are identity experts: they get no row in any expert's stretch
//                    (chosen = -1) and their shares are added up in identity_share[t] for ts_moe_combine.
//   ts_moe_arrange   (token, choice) pairs sorted by expert: every CTA takes the exclusive scan of the
//                    counts and places its pairs behind their expert's offset.  Which row of an
//                    expert's stretch a pair lands in is not fixed; no result depends on it.
//   ts_moe_linear    grouped product over the sorted pairs: row i of expert e's stretch times W_e^T,
//                    W [experts, N, K].  Tiles of 32 pairs x 64 columns, FFMA with float32 sums over k
//                    in ascending order (a pair's result does not depend on its row or on the batch).
//                    With `gated`, W_e holds gate rows then up rows and the epilogue applies the gated
//                    activation (the kinds are listed below) before it stores.  Without `gated`, `unary` 1
//                    stores relu(s)^2 and `row_scale` (one factor a pair) multiplies the sum first: an
//                    expert whose input is weighted, since W (c x) = c (W x).  Input rows are
//                    gathered by token for the first product; the second reads the sorted rows.
//                    A step of up to 64 pairs takes a weight-streaming kernel instead (further down); large
//                    bfloat16 steps may be given to the library's grouped product by the caller.
//   ts_moe_combine   out[t] = sum_j share[t, j] * y[row of (t, j)] (+ the shared expert's output), in the
//                    order of j, float32, rounded once.  Without `share` every weight is 1.  With
//                    `identity_share`, identity_share[t] * x[t] is added (the identity experts' part).
#include "common.cuh"

// the kinds of gated activation are those of common.cuh (ts_gated_activation)

__global__ void moe_route_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                 const int* __restrict__ seq_of_token, int* __restrict__ chosen, float* __restrict__ share,
                                 int* __restrict__ counts, int num_tokens, int experts, int top, int scoring) {
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= num_tokens) return;
    const int lane = threadIdx.x & 31;
    if (seq_of_token && seq_of_token[t] < 0) {            // a padding row takes part in nothing
        for (int j = lane; j < top; j += 32) chosen[(long long)t * top + j] = -1;
        return;
    }
    const float* z = logits + (long long)t * experts;
    float first = 0.f, total = 0.f;
    unsigned long long taken_lo = 0;                       // experts this lane has given away (its e = lane + 32 i, i < 64)
    for (int j = 0; j < top; ++j) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int e = lane, i = 0; e < experts; e += 32, ++i) {
            if (taken_lo >> i & 1) continue;
            const float x = z[e] + (bias ? bias[e] : 0.f);
            if (x > best || (x == best && e < arg)) { best = x; arg = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (arg != 0x7fffffff && (arg & 31) == lane) taken_lo |= 1ull << (arg >> 5);
        if (j == 0) first = best;
        const float w = scoring == 1 ? 1.f / (1.f + expf(-best)) : expf(best - first);   // the first choice is the largest
        total += w;
        if (lane == 0) {
            chosen[(long long)t * top + j] = arg;
            share[(long long)t * top + j] = w;
            atomicAdd(counts + arg, 1);
        }
    }
    __syncwarp();
    if (lane == 0 && scoring == 0)
        for (int j = 0; j < top; ++j) share[(long long)t * top + j] /= total;
}

TS_API int ts_moe_route(const float* logits, const float* bias, const int* seq_of_token, int* chosen, float* share,
                        int* counts, int num_tokens, int experts, int top, int scoring, cudaStream_t stream) {
    TS_REQUIRE(experts > 0 && top > 0 && top <= experts, "moe_route: %d of %d experts", top, experts);
    TS_REQUIRE(experts <= 2048, "moe_route: %d experts are not supported (up to 2048)", experts);
    if (num_tokens <= 0) return 0;
    moe_route_kernel<<<(num_tokens + 3) / 4, 128, 0, stream>>>(logits, bias, seq_of_token, chosen, share, counts,
                                                               num_tokens, experts, top, scoring);
    TS_LAUNCH_CHECK("moe_route");
    return 0;
}

// Scores over all router outputs, choice inside the best groups (see the head of this file).  A warp a token.
// The scores and the choice scores are computed once into the warp's shared memory; every round of a choice
// (the best group, the best output) is a walk of each lane over its own entries and two warp reductions: the
// largest value as an ordered integer, then the lowest index among the lanes that hold it.
__device__ __forceinline__ unsigned ordered_key(float x) {
    const unsigned u = __float_as_uint(x + 0.f);          // -0 becomes +0: equal values, equal keys
    return u & 0x80000000u ? ~u : u | 0x80000000u;
}

// (value, index) of the largest value over the warp, ties to the lower index; index 0x7fffffff: no lane had one
__device__ __forceinline__ int warp_argmax(float best, int arg) {
    const unsigned key = arg == 0x7fffffff ? 0u : ordered_key(best);
    const unsigned top = __reduce_max_sync(0xffffffffu, key);
    return (int)__reduce_min_sync(0xffffffffu, (unsigned)(key == top ? arg : 0x7fffffff));
}

__global__ void moe_route_grouped_kernel(const float* __restrict__ logits, const float* __restrict__ correction,
                                         const int* __restrict__ seq_of_token, int* __restrict__ chosen,
                                         float* __restrict__ share, int* __restrict__ counts, float* __restrict__ identity_share,
                                         int num_tokens, int outputs, int real_experts, int top, int groups, int keep,
                                         float weight_scale, float share_eps) {
    extern __shared__ float route_smem[];                 // per warp: scores, choice scores, groups' ranks, groups' flags
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= num_tokens) return;
    if (seq_of_token && seq_of_token[t] < 0) {            // a padding row takes part in nothing
        for (int j = lane; j < top; j += 32) chosen[(long long)t * top + j] = -1;
        if (lane == 0 && identity_share) identity_share[t] = 0.f;
        return;
    }
    float* score = route_smem + (size_t)warp * 2 * (outputs + groups);
    float* choice = score + outputs;
    float* rank = choice + outputs;
    int* kept = reinterpret_cast<int*>(rank + groups);
    const float* z = logits + (long long)t * outputs;
    float zmax = -INFINITY;
    for (int e = lane; e < outputs; e += 32) zmax = fmaxf(zmax, z[e]);
    zmax = warp_max(zmax);
    float sum = 0.f;
    for (int e = lane; e < outputs; e += 32) {
        const float x = expf(z[e] - zmax);
        score[e] = x;
        sum += x;
    }
    const float inv_sum = 1.f / warp_sum(sum);
    for (int e = lane; e < outputs; e += 32) {
        const float x = score[e] * inv_sum;
        score[e] = x;
        choice[e] = x + (correction ? correction[e] : 0.f);
    }
    __syncwarp();
    const int per = outputs / groups;
    if (keep < groups) {
        for (int g = lane; g < groups; g += 32) {
            float m = -INFINITY;
            for (int e = g * per; e < (g + 1) * per; ++e) m = fmaxf(m, choice[e]);
            rank[g] = m;
            kept[g] = 0;
        }
        __syncwarp();
        for (int r = 0; r < keep; ++r) {                  // the best group not kept yet; ties go to the lower index
            float best = -INFINITY;
            int arg = 0x7fffffff;
            for (int g = lane; g < groups; g += 32) {
                if (kept[g]) continue;
                const float x = rank[g];
                if (arg == 0x7fffffff || x > best) { best = x; arg = g; }
            }
            arg = warp_argmax(best, arg);
            if (lane == 0 && arg != 0x7fffffff) kept[arg] = 1;
            __syncwarp();
        }
    }
    float total = 0.f, identity = 0.f;
    unsigned long long taken_lo = 0;
    for (int j = 0; j < top; ++j) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int e = lane, i = 0; e < outputs; e += 32, ++i) {
            if (taken_lo >> i & 1) continue;
            if (keep < groups && !kept[e / per]) continue;
            const float x = choice[e];
            if (arg == 0x7fffffff || x > best) { best = x; arg = e; }
        }
        arg = warp_argmax(best, arg);
        if (arg == 0x7fffffff) {                           // fewer outputs allowed than `top`: the choice stays empty
            if (lane == 0) { chosen[(long long)t * top + j] = -1; share[(long long)t * top + j] = 0.f; }
            continue;
        }
        if ((arg & 31) == lane) taken_lo |= 1ull << (arg >> 5);
        const float w = score[arg];
        total += w;
        const bool real = arg < real_experts;
        if (!real) identity += w;
        if (lane == 0) {
            chosen[(long long)t * top + j] = real ? arg : -1;
            share[(long long)t * top + j] = w;
            if (real) atomicAdd(counts + arg, 1);
        }
    }
    __syncwarp();
    const float norm = weight_scale / (total + share_eps);
    if (lane == 0) {
        for (int j = 0; j < top; ++j) share[(long long)t * top + j] *= norm;
        if (identity_share) identity_share[t] = identity * norm;
    }
}

TS_API int ts_moe_route_grouped(const float* logits, const float* correction, const int* seq_of_token, int* chosen,
                                float* share, int* counts, float* identity_share, int num_tokens, int outputs,
                                int real_experts, int top, int groups, int keep, float weight_scale, float share_eps,
                                cudaStream_t stream) {
    TS_REQUIRE(outputs > 0 && top > 0 && top <= outputs && real_experts >= 0 && real_experts <= outputs,
               "moe_route: %d of %d router outputs, %d of them experts", top, outputs, real_experts);
    TS_REQUIRE(outputs <= 2048, "moe_route: %d router outputs are not supported (up to 2048)", outputs);
    TS_REQUIRE(groups > 0 && outputs % groups == 0 && keep > 0 && keep <= groups && groups <= 1024,
               "moe_route: %d outputs in %d groups of which %d are kept", outputs, groups, keep);
    TS_REQUIRE(real_experts == outputs || identity_share, "moe_route: identity experts need a place for their shares");
    if (num_tokens <= 0) return 0;
    const size_t per_warp = (size_t)2 * (outputs + groups) * sizeof(float);           // at most 24 KB
    const int warps = per_warp * 4 <= 48 * 1024 ? 4 : 2;
    moe_route_grouped_kernel<<<(num_tokens + warps - 1) / warps, 32 * warps, per_warp * warps, stream>>>(logits, correction, seq_of_token, chosen, share,
                                                                        counts, identity_share, num_tokens, outputs,
                                                                        real_experts, top, groups, keep, weight_scale,
                                                                        share_eps);
    TS_LAUNCH_CHECK("moe_route_grouped");
    return 0;
}

// offsets[e] = pairs of experts before e (offsets[experts] = all); row_of_pair / pair_of_row both ways.
__global__ void moe_arrange_kernel(const int* __restrict__ chosen, const int* __restrict__ counts, int* __restrict__ cursor,
                                   int* __restrict__ offsets, int* __restrict__ pair_of_row, int* __restrict__ row_of_pair,
                                   int pairs, int experts) {
    extern __shared__ int start[];                        // experts + 1
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < experts; ++e) { start[e] = run; run += counts[e]; }
        start[experts] = run;
    }
    __syncthreads();
    if (blockIdx.x == 0)
        for (int e = threadIdx.x; e <= experts; e += blockDim.x) offsets[e] = start[e];
    for (int p = blockIdx.x * blockDim.x + threadIdx.x; p < pairs; p += gridDim.x * blockDim.x) {
        const int e = chosen[p];
        if (e < 0) { row_of_pair[p] = -1; continue; }
        const int row = start[e] + atomicAdd(cursor + e, 1);
        pair_of_row[row] = p;
        row_of_pair[p] = row;
    }
}

TS_API int ts_moe_arrange(const int* chosen, const int* counts, int* cursor, int* offsets, int* pair_of_row,
                          int* row_of_pair, int pairs, int experts, cudaStream_t stream) {
    if (pairs <= 0) return 0;
    const int blocks = min((pairs + 255) / 256, 148);
    moe_arrange_kernel<<<blocks, 256, (experts + 1) * sizeof(int), stream>>>(chosen, counts, cursor, offsets, pair_of_row,
                                                                           row_of_pair, pairs, experts);
    TS_LAUNCH_CHECK("moe_arrange");
    return 0;
}

constexpr int GM = 32, GN = 64, GK = 16;

template <typename T, bool GATED>
__global__ void __launch_bounds__(256)
moe_linear_kernel(const T* __restrict__ x, long long x_stride, const int* __restrict__ pair_of_row, int top,
                  const int* __restrict__ offsets, int experts, const T* __restrict__ w, int N, int K, T* __restrict__ y,
                  int out_cols, int kind, float limit, float alpha, const float* __restrict__ row_scale, int unary) {
    __shared__ float As[GK][GM + 1];
    __shared__ float Bs[GK][GN + 1];
    __shared__ float Us[GATED ? GK : 1][GN + 1];
    __shared__ int rows_src[GM];
    // which expert's stretch this row tile belongs to: tiles are numbered expert by expert
    int tile = blockIdx.y, e = 0, first = 0, last = 0;
    for (; e < experts; ++e) {
        first = offsets[e]; last = offsets[e + 1];
        const int tiles = (last - first + GM - 1) / GM;
        if (tile < tiles) break;
        tile -= tiles;
    }
    if (e == experts) return;
    const int row0 = first + tile * GM;
    const int nrows = min(GM, last - row0);
    const int col0 = blockIdx.x * GN;
    const int tid = threadIdx.x;
    __shared__ float rows_scale[GM];
    if (tid < GM) {
        int src = -1;
        float c = 1.f;
        if (tid < nrows) {
            const int pair = pair_of_row ? pair_of_row[row0 + tid] : row0 + tid;
            src = pair_of_row ? pair / top : pair;
            if (row_scale) c = row_scale[pair];
        }
        rows_src[tid] = src;
        rows_scale[tid] = c;
    }
    __syncthreads();
    const T* we = w + (long long)e * N * K;
    const int half = GATED ? N / 2 : 0;                   // gate rows [0, half), up rows [half, N)
    const int tr = (tid / 16) * 2, tc = (tid % 16) * 4;   // 2 x 4 outputs a thread
    float acc[2][4], accu[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = accu[i][j] = 0.f;
    const int lk = tid % GK, lr = tid / GK;               // 16 rows of loads a pass
    for (int k0 = 0; k0 < K; k0 += GK) {
        const int gk = k0 + lk;
#pragma unroll
        for (int i = 0; i < GM / 16; ++i) {
            const int r = lr + 16 * i;
            const int src = rows_src[r];
            As[lk][r] = (src >= 0 && gk < K) ? to_float<T>(x[(long long)src * x_stride + gk]) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < GN / 16; ++i) {
            const int c = lr + 16 * i;
            const int gc = col0 + c;
            const bool in = gc < (GATED ? half : N) && gk < K;
            Bs[lk][c] = in ? to_float<T>(we[(long long)gc * K + gk]) : 0.f;
            if (GATED) Us[lk][c] = in ? to_float<T>(we[(long long)(half + gc) * K + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < GK; ++k) {
            float a[2], b[4], u[4];
#pragma unroll
            for (int i = 0; i < 2; ++i) a[i] = As[k][tr + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) { b[j] = Bs[k][tc + j]; if (GATED) u[j] = Us[k][tc + j]; }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
                    if (GATED) accu[i][j] = fmaf(a[i], u[j], accu[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        if (tr + i >= nrows) continue;
        T* dst = y + (long long)(row0 + tr + i) * out_cols;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gc = col0 + tc + j;
            if (gc >= out_cols) continue;
            float v = GATED ? ts_gated_activation(kind, acc[i][j], accu[i][j], limit, alpha) : acc[i][j] * rows_scale[tr + i];
            if (!GATED && unary == 1) v = fmaxf(v, 0.f) * fmaxf(v, 0.f);
            dst[gc] = from_float<T>(v);
        }
    }
}

// The same product for a step of a few tokens (decoding): a row tile is up to 8 pairs of one expert,
// kept in shared memory; a warp owns output columns and streams their weight rows once, 16 bytes a
// lane at a time, for all rows of the tile at once.  A row's sum over k has one order, whatever the batch.
constexpr int SR = 8, SWARPS = 8;

template <typename T, bool GATED>
__global__ void __launch_bounds__(SWARPS * 32)
moe_linear_rows_kernel(const T* __restrict__ x, long long x_stride, const int* __restrict__ pair_of_row, int top,
                       const int* __restrict__ offsets, int experts, const T* __restrict__ w, int N, int K,
                       T* __restrict__ y, int out_cols, int cols_per_cta, int kind, float limit, float alpha,
                       const float* __restrict__ row_scale, int unary) {
    extern __shared__ __align__(16) unsigned char raw[];
    __shared__ float rows_scale[SR];
    T* xs = reinterpret_cast<T*>(raw);                    // [SR][K]
    constexpr int VN = 16 / sizeof(T);
    // Which expert's stretch this row tile belongs to (tiles are numbered expert by expert): every warp looks at 32
    // experts at a time, a lane an expert, and a scan over the lanes' tile counts finds the one; walking the
    // offsets one dependent load after the other cost the last experts' CTAs some thousand cycles before their first byte.
    int tile = blockIdx.y, e = experts, first = 0, last = 0;
    {
        const int ln = threadIdx.x & 31;
        for (int e0 = 0; e0 < experts; e0 += 32) {
            const int le = e0 + ln;
            const int f = le < experts ? offsets[le] : 0, l = le < experts ? offsets[le + 1] : 0;
            const int tiles = le < experts ? (l - f + SR - 1) / SR : 0;
            int incl = tiles;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (ln >= o) incl += v;
            }
            const unsigned hit = __ballot_sync(0xffffffffu, tile < incl);
            if (hit) {
                const int src = __ffs(hit) - 1;
                e = e0 + src;
                first = __shfl_sync(0xffffffffu, f, src);
                last = __shfl_sync(0xffffffffu, l, src);
                tile -= __shfl_sync(0xffffffffu, incl - tiles, src);
                break;
            }
            tile -= __shfl_sync(0xffffffffu, incl, 31);
        }
    }
    if (e == experts) return;
    const int row0 = first + tile * SR;
    const int nrows = min(SR, last - row0);
    for (int i = threadIdx.x; i < SR * (K / VN); i += blockDim.x) {
        const int r = i / (K / VN), c = i % (K / VN);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < nrows) {
            const int src = pair_of_row ? pair_of_row[row0 + r] / top : row0 + r;
            v = *reinterpret_cast<const uint4*>(x + (long long)src * x_stride + c * VN);
        }
        *reinterpret_cast<uint4*>(xs + (long long)r * K + c * VN) = v;
    }
    if (threadIdx.x < SR) {
        float c = 1.f;
        if (row_scale && (int)threadIdx.x < nrows) c = row_scale[pair_of_row ? pair_of_row[row0 + threadIdx.x] : row0 + threadIdx.x];
        rows_scale[threadIdx.x] = c;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* we = w + (long long)e * N * K;
    const int half = GATED ? N / 2 : 0;
    const int col_end = min(out_cols, (int)(blockIdx.x + 1) * cols_per_cta);
    // A warp takes CG columns at a time: their weight rows are independent streams, so CG (twice that with a gate)
    // 16-byte loads a lane are under way at once instead of one column's after the other's.  A row's sum over k has
    // the same order as with one column at a time.
    constexpr int CG = GATED ? 2 : 4;
    for (int base = blockIdx.x * cols_per_cta + warp * CG; base < col_end; base += SWARPS * CG) {
        float acc[CG][SR], accu[GATED ? CG : 1][SR];
#pragma unroll
        for (int g = 0; g < CG; ++g)
#pragma unroll
            for (int r = 0; r < SR; ++r) { acc[g][r] = 0.f; if (GATED) accu[g][r] = 0.f; }
#pragma unroll 2
        for (int c = lane * VN; c < K; c += 32 * VN) {
            uint4 wv[CG], uv[GATED ? CG : 1];
#pragma unroll
            for (int g = 0; g < CG; ++g) {
                const int col = min(base + g, col_end - 1);           // a column past the end: loaded again, not stored
                wv[g] = *reinterpret_cast<const uint4*>(we + (long long)col * K + c);
                if (GATED) uv[g] = *reinterpret_cast<const uint4*>(we + (long long)(half + col) * K + c);
            }
#pragma unroll
            for (int r = 0; r < SR; ++r) {
                if (r >= nrows) break;                    // a decoding step often gives an expert one pair
                const uint4 xv = *reinterpret_cast<const uint4*>(xs + (long long)r * K + c);
                const T* xl = reinterpret_cast<const T*>(&xv);
#pragma unroll
                for (int g = 0; g < CG; ++g) {
                    const T* wl = reinterpret_cast<const T*>(&wv[g]);
                    const T* ul = reinterpret_cast<const T*>(&uv[GATED ? g : 0]);
#pragma unroll
                    for (int i = 0; i < VN; ++i) {
                        const float xf = to_float<T>(xl[i]);
                        acc[g][r] = fmaf(xf, to_float<T>(wl[i]), acc[g][r]);
                        if (GATED) accu[g][r] = fmaf(xf, to_float<T>(ul[i]), accu[g][r]);
                    }
                }
            }
        }
#pragma unroll
        for (int g = 0; g < CG; ++g) {
            const int col = base + g;
            if (col >= col_end) break;                    // the same for the whole warp
#pragma unroll
            for (int r = 0; r < SR; ++r) {
                if (r >= nrows) break;                    // the same for the whole CTA: no lane is left out of a sum
                const float gsum = warp_sum(acc[g][r]);
                const float usum = GATED ? warp_sum(accu[GATED ? g : 0][r]) : 0.f;
                if (lane == 0) {
                    float v = GATED ? ts_gated_activation(kind, gsum, usum, limit, alpha) : gsum * rows_scale[r];
                    if (!GATED && unary == 1) v = fmaxf(v, 0.f) * fmaxf(v, 0.f);
                    y[(long long)(row0 + r) * out_cols + col] = from_float<T>(v);
                }
            }
        }
    }
}

TS_API int ts_moe_linear(const void* x, long long x_stride, const int* pair_of_row, int top, const int* offsets,
                         int experts, const void* w, int N, int K, void* y, int pairs, int gated, int kind, float limit,
                         float alpha, const float* row_scale, int unary, int dtype, cudaStream_t stream) {
    TS_REQUIRE(experts > 0 && N > 0 && K > 0 && top > 0, "moe_linear: bad sizes");
    TS_REQUIRE(!gated || (!row_scale && !unary), "moe_linear: a gated product takes no row scale and no other activation");
    TS_REQUIRE(!gated || N % 2 == 0, "moe_linear: a gated weight holds gate and up rows of equal number");
    if (pairs <= 0) return 0;
    const int out_cols = gated ? N / 2 : N;
    const int elem = dtype == TS_F32 ? 4 : 2, vn = 16 / elem;
    if (pairs <= 64 && K % vn == 0 && (x_stride * elem) % 16 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0 &&
        (size_t)SR * K * elem <= 200 * 1024 && (dtype == TS_F32 || dtype == TS_BF16)) {
        const int tiles = (pairs + SR - 1) / SR + experts;
        const int cols_per_cta = out_cols <= 256 ? 32 : 64;
        dim3 sgrid((out_cols + cols_per_cta - 1) / cols_per_cta, tiles);
        const size_t smem = (size_t)SR * K * elem;
#define TS_MOE_ROWS(TYPE, G)                                                                                           \
        do {                                                                                                           \
            if (smem > 48 * 1024)                                                                                      \
                cudaFuncSetAttribute(moe_linear_rows_kernel<TYPE, G>, cudaFuncAttributeMaxDynamicSharedMemorySize,     \
                                     (int)smem);                                                                       \
            moe_linear_rows_kernel<TYPE, G><<<sgrid, SWARPS * 32, smem, stream>>>(                                     \
                (const TYPE*)x, x_stride, pair_of_row, top, offsets, experts, (const TYPE*)w, N, K, (TYPE*)y, out_cols, \
                cols_per_cta, kind, limit, alpha, row_scale, unary);                                                                  \
        } while (0)
        if (dtype == TS_F32) { if (gated) TS_MOE_ROWS(float, true); else TS_MOE_ROWS(float, false); }
        else { if (gated) TS_MOE_ROWS(__nv_bfloat16, true); else TS_MOE_ROWS(__nv_bfloat16, false); }
#undef TS_MOE_ROWS
        TS_LAUNCH_CHECK("moe_linear");
        return 0;
    }
    const int row_tiles = (pairs + GM - 1) / GM + experts;       // every expert may end in a ragged tile
    TS_REQUIRE(row_tiles <= 65535, "moe_linear: %d pairs need more than 65535 row tiles", pairs);
    dim3 grid((out_cols + GN - 1) / GN, row_tiles);
#define TS_MOE_LINEAR(TYPE, G)                                                                                       \
    moe_linear_kernel<TYPE, G><<<grid, 256, 0, stream>>>((const TYPE*)x, x_stride, pair_of_row, top, offsets, experts, \
                                                         (const TYPE*)w, N, K, (TYPE*)y, out_cols, kind, limit, alpha, \
                                                         row_scale, unary)
    if (dtype == TS_F32) { if (gated) TS_MOE_LINEAR(float, true); else TS_MOE_LINEAR(float, false); }
    else if (dtype == TS_BF16) { if (gated) TS_MOE_LINEAR(__nv_bfloat16, true); else TS_MOE_LINEAR(__nv_bfloat16, false); }
    else return ts_fail("moe_linear: unknown dtype code %d", dtype);
#undef TS_MOE_LINEAR
    TS_LAUNCH_CHECK("moe_linear");
    return 0;
}

template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ y, const int* __restrict__ row_of_pair,
                                   const float* __restrict__ share, const T* __restrict__ shared_out, T* __restrict__ out,
                                   int width, int top, const T* __restrict__ x, const float* __restrict__ identity_share) {
    const long long t = blockIdx.x;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float s = 0.f;
        for (int j = 0; j < top; ++j) {
            const int row = row_of_pair[t * top + j];
            if (row >= 0) s = fmaf(share ? share[t * top + j] : 1.f, to_float<T>(y[(long long)row * width + i]), s);
        }
        if (shared_out) s += to_float<T>(shared_out[t * width + i]);
        if (identity_share) s = fmaf(identity_share[t], to_float<T>(x[t * width + i]), s);
        out[t * width + i] = from_float<T>(s);
    }
}

TS_API int ts_moe_combine(const void* y, const int* row_of_pair, const float* share, const void* shared_out, void* out,
                          int num_tokens, int width, int top, int dtype, const void* x, const float* identity_share,
                          cudaStream_t stream) {
    TS_REQUIRE(!identity_share || x, "moe_combine: identity experts need the experts' input");
    if (num_tokens <= 0) return 0;
    if (dtype == TS_F32)
        moe_combine_kernel<float><<<num_tokens, 128, 0, stream>>>((const float*)y, row_of_pair, share,
                                                                  (const float*)shared_out, (float*)out, width, top,
                                                                  (const float*)x, identity_share);
    else if (dtype == TS_BF16)
        moe_combine_kernel<__nv_bfloat16><<<num_tokens, 128, 0, stream>>>((const __nv_bfloat16*)y, row_of_pair, share,
            (const __nv_bfloat16*)shared_out, (__nv_bfloat16*)out, width, top, (const __nv_bfloat16*)x, identity_share);
    else
        return ts_fail("moe_combine: unknown dtype code %d", dtype);
    TS_LAUNCH_CHECK("moe_combine");
    return 0;
}

// out[t, i] = activation(gate_up[t, i], gate_up[t, I + i]) for the kinds above (dense layers and the shared expert).
template <typename T>
__global__ void gated_activation_kernel(const T* __restrict__ gate_up, T* __restrict__ out, long long total, int inter,
                                        int kind, float limit, float alpha) {
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long t = idx / inter;
        const int i = (int)(idx % inter);
        const float g = to_float<T>(gate_up[t * 2 * inter + i]);
        const float u = to_float<T>(gate_up[t * 2 * inter + inter + i]);
        out[idx] = from_float<T>(ts_gated_activation(kind, g, u, limit, alpha));
    }
}

TS_API int ts_gated_activation(const void* gate_up, void* out, int num_tokens, int inter, int kind, float limit,
                               float alpha, int dtype, cudaStream_t stream) {
    TS_REQUIRE(num_tokens >= 0 && inter > 0 && kind >= 0 && kind <= TS_ACT_LAST, "gated_activation: bad arguments");
    if (num_tokens == 0) return 0;
    const long long total = (long long)num_tokens * inter;
    const unsigned blocks = (unsigned)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    if (dtype == TS_F32)
        gated_activation_kernel<float><<<blocks, 256, 0, stream>>>((const float*)gate_up, (float*)out, total, inter, kind,
                                                                   limit, alpha);
    else if (dtype == TS_BF16)
        gated_activation_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)gate_up,
                                                                           (__nv_bfloat16*)out, total, inter, kind, limit, alpha);
    else
        return ts_fail("gated_activation: unknown dtype code %d", dtype);
    TS_LAUNCH_CHECK("gated_activation");
    return 0;
}

// out[r, c] = act(x[r, c] * scale[pair of sorted row r]) for the ungated activations (after a library product).
// VEC: 16 bytes a thread (the row width is a multiple of that many elements and the pointers are aligned).
template <typename T, bool VEC>
__global__ void row_scaled_activation_kernel(const T* __restrict__ x, const int* __restrict__ pair_of_row,
                                             const float* __restrict__ row_scale, T* __restrict__ out, long long total,
                                             int cols, int unary) {
    constexpr int VN = VEC ? 16 / (int)sizeof(T) : 1;
    for (long long idx = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * VN; idx < total;
         idx += (long long)gridDim.x * blockDim.x * VN) {
        const long long r = idx / cols;
        const float c = row_scale ? row_scale[pair_of_row ? pair_of_row[r] : r] : 1.f;
        if (VEC) {
            uint4 raw = *reinterpret_cast<const uint4*>(x + idx);
            T* v = reinterpret_cast<T*>(&raw);
#pragma unroll
            for (int i = 0; i < VN; ++i) {
                float f = to_float<T>(v[i]) * c;
                if (unary == 1) f = fmaxf(f, 0.f) * fmaxf(f, 0.f);
                v[i] = from_float<T>(f);
            }
            *reinterpret_cast<uint4*>(out + idx) = raw;
        } else {
            float f = to_float<T>(x[idx]) * c;
            if (unary == 1) f = fmaxf(f, 0.f) * fmaxf(f, 0.f);
            out[idx] = from_float<T>(f);
        }
    }
}

TS_API int ts_row_scaled_activation(const void* x, const int* pair_of_row, const float* row_scale, void* out, int rows,
                                    int cols, int unary, int dtype, cudaStream_t stream) {
    TS_REQUIRE(rows >= 0 && cols > 0, "row_scaled_activation: bad sizes");
    if (rows == 0) return 0;
    const long long total = (long long)rows * cols;
    const int elem = dtype == TS_F32 ? 4 : 2, vn = 16 / elem;
    const bool vec = cols % vn == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)out % 16 == 0;
    const long long threads = vec ? total / vn : total;
    const unsigned blocks = (unsigned)((threads + 255) / 256 < 148 * 16 ? (threads + 255) / 256 : 148 * 16);
#define TS_ROW_SCALED(TYPE)                                                                                         \
    do {                                                                                                            \
        if (vec) row_scaled_activation_kernel<TYPE, true><<<blocks, 256, 0, stream>>>(                              \
            (const TYPE*)x, pair_of_row, row_scale, (TYPE*)out, total, cols, unary);                                \
        else row_scaled_activation_kernel<TYPE, false><<<blocks, 256, 0, stream>>>(                                 \
            (const TYPE*)x, pair_of_row, row_scale, (TYPE*)out, total, cols, unary);                                \
    } while (0)
    if (dtype == TS_F32) TS_ROW_SCALED(float);
    else if (dtype == TS_BF16) TS_ROW_SCALED(__nv_bfloat16);
    else return ts_fail("row_scaled_activation: unknown dtype code %d", dtype);
#undef TS_ROW_SCALED
    TS_LAUNCH_CHECK("row_scaled_activation");
    return 0;
}
