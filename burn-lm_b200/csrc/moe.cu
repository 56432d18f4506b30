// Mixture of experts for a packed step: router, grouping of the (token, expert) pairs by expert, the experts'
// gated feed-forwards as grouped products over the pairs in that order, and the sum per token.
//
//   z = W_router h (fp32), s = sigmoid(z); a token takes its `top` experts of largest s (ties: the lower index)
//   with weight s (not renormalised).  weight_on_input: out = sum_k expert_k(s_k h); else out = sum_k s_k expert_k(h).
//   expert(x) = W_down (silu(W_gate x) * (W_up x)).
//
// Everything runs on the device with sizes that depend on the step's token count only, so a step can be captured
// in a CUDA graph: the grids cover the worst case (every expert's share padded to a tile) and blocks beyond the
// real tiles return.
#include "common.cuh"

BLM_API const char* blm_moe_last_error() { return g_blm_error; }

// ---------------------------------------------------------------------------------------------
// router: one block per token
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void moe_route_kernel(const T* __restrict__ h, const float* __restrict__ router, int width, int n_experts, int top,
                                 int* __restrict__ ids, float* __restrict__ weights) {
    extern __shared__ float smem[];
    float* x = smem;                 // [width]
    float* score = smem + width;     // [n_experts]
    const int n = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    for (int d = threadIdx.x; d < width; d += blockDim.x) x[d] = to_f32(h[(size_t)n * width + d]);
    __syncthreads();
    for (int e = warp; e < n_experts; e += n_warps) {
        const float* w = router + (size_t)e * width;
        float z = 0.f;
        for (int d = lane; d < width; d += 32) z = fmaf(w[d], x[d], z);
        z = warp_sum(z);
        if (lane == 0) score[e] = 1.0f / (1.0f + expf(-z));
    }
    __syncthreads();
    if (warp == 0) {
        for (int k = 0; k < top; ++k) {
            float best = -1.f;
            int arg = 0x7fffffff;
            for (int e = lane; e < n_experts; e += 32) {
                const float s = score[e];
                if (s > best) { best = s; arg = e; }     // ascending e per lane: the lower index stays on a tie
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
                if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
            }
            if (lane == 0) {
                ids[(size_t)n * top + k] = arg;
                weights[(size_t)n * top + k] = best;
                score[arg] = -2.f;                       // taken
            }
            __syncwarp();
        }
    }
}

BLM_API int blm_moe_route(const void* h, int dtype, const float* router, int n_tokens, int width, int n_experts, int top, int* ids,
                          float* weights, cudaStream_t stream) {
    if (n_tokens == 0) return BLM_OK;
    BLM_REQUIRE(n_tokens > 0 && width > 0 && n_experts > 0 && top > 0 && top <= n_experts, "moe_route: bad sizes");
    const size_t smem = ((size_t)width + n_experts) * sizeof(float);
    BLM_REQUIRE(smem <= 48 * 1024, "moe_route: width %d and %d experts need %zu bytes of shared memory", width, n_experts, smem);
    if (dtype == BLM_F32)
        moe_route_kernel<float><<<n_tokens, 128, smem, stream>>>((const float*)h, router, width, n_experts, top, ids, weights);
    else if (dtype == BLM_BF16)
        moe_route_kernel<__nv_bfloat16><<<n_tokens, 128, smem, stream>>>((const __nv_bfloat16*)h, router, width, n_experts, top, ids, weights);
    else
        return blm_fail(BLM_BAD_ARGUMENT, "moe_route: dtype %d", dtype);
    return blm_check_launch("moe_route");
}

// ---------------------------------------------------------------------------------------------
// grouping: offsets[e] .. offsets[e + 1] are the places of expert e's pairs; order[place] = pair (token * top + k);
// place_of[pair] = place.  One block.  The order inside an expert's share is whatever the atomics give: every
// pair's row is computed on its own, so no result depends on it.
// ---------------------------------------------------------------------------------------------
__global__ void moe_group_kernel(const int* __restrict__ ids, int n_pairs, int n_experts, int* __restrict__ offsets,
                                 int* __restrict__ order, int* __restrict__ place_of) {
    extern __shared__ int counts[];      // [n_experts] counts, then [n_experts] cursors
    int* cursor = counts + n_experts;
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int a = threadIdx.x; a < n_pairs; a += blockDim.x) atomicAdd(&counts[ids[a]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < n_experts; ++e) {
            offsets[e] = run;
            cursor[e] = run;
            run += counts[e];
        }
        offsets[n_experts] = run;
    }
    __syncthreads();
    for (int a = threadIdx.x; a < n_pairs; a += blockDim.x) {
        const int place = atomicAdd(&cursor[ids[a]], 1);
        order[place] = a;
        place_of[a] = place;
    }
}

BLM_API int blm_moe_group(const int* ids, int n_pairs, int n_experts, int* offsets, int* order, int* place_of, cudaStream_t stream) {
    if (n_pairs == 0) return BLM_OK;
    BLM_REQUIRE(n_pairs > 0 && n_experts > 0 && n_experts <= 4096, "moe_group: bad sizes");
    moe_group_kernel<<<1, 1024, 2 * (size_t)n_experts * sizeof(int), stream>>>(ids, n_pairs, n_experts, offsets, order, place_of);
    return blm_check_launch("moe_group");
}

// ---------------------------------------------------------------------------------------------
// grouped products on the CUDA cores (fp32 sums): tiles of kBM places x kBN outputs, the reduction in slices of
// kBK.  A block finds the expert and the places of its tile from the offsets; blocks beyond the last tile return.
// ---------------------------------------------------------------------------------------------
constexpr int kBM = 32, kBN = 32, kBK = 32;

__device__ __forceinline__ bool moe_find_tile(const int* __restrict__ offsets, int n_experts, int tile, int* expert, int* first, int* last) {
    __shared__ int found[3];
    if (threadIdx.x == 0) {
        int t = tile, e = 0;
        found[0] = -1;
        for (; e < n_experts; ++e) {
            const int begin = offsets[e], end = offsets[e + 1];
            const int tiles = (end - begin + kBM - 1) / kBM;
            if (t < tiles) {
                found[0] = e;
                found[1] = begin + t * kBM;
                found[2] = end;
                break;
            }
            t -= tiles;
        }
    }
    __syncthreads();
    *expert = found[0];
    *first = found[1];
    *last = found[2];
    return found[0] >= 0;
}

// x rounded as the activations' dtype rounds it: the input of a product in that dtype
template <typename T> __device__ __forceinline__ float as_input(float v) { return to_f32(from_f32<T>(v)); }

// act[place, c] = silu(x . Wgate[e, c]) * (x . Wup[e, c]),  x = the pair's token row of h (times the pair's weight when
// `scale_input`).  w_gu: [experts, 2 ff, width], an expert's gate rows followed by its up rows.
template <typename T>
__global__ void moe_gate_up_kernel(const T* __restrict__ h, const float* __restrict__ weights, const int* __restrict__ order,
                                   const int* __restrict__ offsets, const T* __restrict__ w_gu, T* __restrict__ act, int width, int ff,
                                   int n_experts, int top, int scale_input) {
    __shared__ float xs[kBM][kBK + 1], gs[kBN][kBK + 1], us[kBN][kBK + 1];
    __shared__ int token_of[kBM];
    __shared__ float scale_of[kBM];
    int e, first, last;
    if (!moe_find_tile(offsets, n_experts, blockIdx.x, &e, &first, &last)) return;
    const int c0 = blockIdx.y * kBN;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;       // 16 x 16 threads, 2 places x 2 outputs each
    if (threadIdx.x < kBM) {
        const int place = first + threadIdx.x;
        int tok = -1;
        float sc = 1.f;
        if (place < last) {
            const int pair = order[place];
            tok = pair / top;
            if (scale_input) sc = weights[pair];
        }
        token_of[threadIdx.x] = tok;
        scale_of[threadIdx.x] = sc;
    }
    __syncthreads();
    const T* wg = w_gu + (size_t)e * 2 * ff * width;
    const T* wu = wg + (size_t)ff * width;
    float ag[2][2] = {{0.f, 0.f}, {0.f, 0.f}}, au[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    for (int k0 = 0; k0 < width; k0 += kBK) {
        for (int idx = threadIdx.x; idx < kBM * kBK; idx += blockDim.x) {
            const int r = idx / kBK, kk = idx % kBK, k = k0 + kk;
            const int tok = token_of[r];
            float v = 0.f;
            if (tok >= 0 && k < width) {
                v = to_f32(h[(size_t)tok * width + k]);
                if (scale_input) v = as_input<T>(scale_of[r] * v);
            }
            xs[r][kk] = v;
        }
        for (int idx = threadIdx.x; idx < kBN * kBK; idx += blockDim.x) {
            const int r = idx / kBK, kk = idx % kBK, k = k0 + kk, c = c0 + r;
            const bool in = c < ff && k < width;
            gs[r][kk] = in ? to_f32(wg[(size_t)c * width + k]) : 0.f;
            us[r][kk] = in ? to_f32(wu[(size_t)c * width + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kBK; ++kk) {
            const float x0 = xs[ty][kk], x1 = xs[ty + 16][kk];
            const float g0 = gs[tx][kk], g1 = gs[tx + 16][kk], u0 = us[tx][kk], u1 = us[tx + 16][kk];
            ag[0][0] = fmaf(x0, g0, ag[0][0]); ag[0][1] = fmaf(x0, g1, ag[0][1]);
            ag[1][0] = fmaf(x1, g0, ag[1][0]); ag[1][1] = fmaf(x1, g1, ag[1][1]);
            au[0][0] = fmaf(x0, u0, au[0][0]); au[0][1] = fmaf(x0, u1, au[0][1]);
            au[1][0] = fmaf(x1, u0, au[1][0]); au[1][1] = fmaf(x1, u1, au[1][1]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int place = first + ty + 16 * i, c = c0 + tx + 16 * j;
            if (place < last && c < ff) {
                const float g = ag[i][j];
                act[(size_t)place * ff + c] = from_f32<T>(g / (1.0f + expf(-g)) * au[i][j]);
            }
        }
}

// y[place, c] = act[place] . Wdown[e, c]   (fp32 out).  w_down: [experts, width, ff].
template <typename T>
__global__ void moe_down_kernel(const T* __restrict__ act, const int* __restrict__ offsets, const T* __restrict__ w_down,
                                float* __restrict__ y, int width, int ff, int n_experts) {
    __shared__ float xs[kBM][kBK + 1], ws[kBN][kBK + 1];
    int e, first, last;
    if (!moe_find_tile(offsets, n_experts, blockIdx.x, &e, &first, &last)) return;
    const int c0 = blockIdx.y * kBN;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const T* wd = w_down + (size_t)e * width * ff;
    float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    for (int k0 = 0; k0 < ff; k0 += kBK) {
        for (int idx = threadIdx.x; idx < kBM * kBK; idx += blockDim.x) {
            const int r = idx / kBK, kk = idx % kBK, k = k0 + kk, place = first + r;
            xs[r][kk] = (place < last && k < ff) ? to_f32(act[(size_t)place * ff + k]) : 0.f;
        }
        for (int idx = threadIdx.x; idx < kBN * kBK; idx += blockDim.x) {
            const int r = idx / kBK, kk = idx % kBK, k = k0 + kk, c = c0 + r;
            ws[r][kk] = (c < width && k < ff) ? to_f32(wd[(size_t)c * ff + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kBK; ++kk) {
            const float x0 = xs[ty][kk], x1 = xs[ty + 16][kk], w0 = ws[tx][kk], w1 = ws[tx + 16][kk];
            acc[0][0] = fmaf(x0, w0, acc[0][0]); acc[0][1] = fmaf(x0, w1, acc[0][1]);
            acc[1][0] = fmaf(x1, w0, acc[1][0]); acc[1][1] = fmaf(x1, w1, acc[1][1]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int place = first + ty + 16 * i, c = c0 + tx + 16 * j;
            if (place < last && c < width) y[(size_t)place * width + c] = acc[i][j];
        }
}

BLM_API int blm_moe_experts(const void* h, int dtype, const float* weights, const int* order, const int* offsets, const void* w_gu,
                            const void* w_down, void* act, float* y, int n_tokens, int width, int ff, int n_experts, int top,
                            int scale_input, cudaStream_t stream) {
    if (n_tokens == 0) return BLM_OK;
    BLM_REQUIRE(n_tokens > 0 && width > 0 && ff > 0 && n_experts > 0 && top > 0, "moe_experts: bad sizes");
    const long long pairs = (long long)n_tokens * top;
    const long long tiles = (pairs + kBM - 1) / kBM + n_experts;      // every expert's share may end in a tile that is not full
    BLM_REQUIRE(tiles < (1ll << 31), "moe_experts: %lld tiles", tiles);
    const dim3 g1((unsigned)tiles, (unsigned)((ff + kBN - 1) / kBN)), g2((unsigned)tiles, (unsigned)((width + kBN - 1) / kBN));
    BLM_REQUIRE(g1.y <= 65535 && g2.y <= 65535, "moe_experts: too many output tiles");
    if (dtype == BLM_F32) {
        moe_gate_up_kernel<float><<<g1, 256, 0, stream>>>((const float*)h, weights, order, offsets, (const float*)w_gu, (float*)act, width,
                                                          ff, n_experts, top, scale_input);
        moe_down_kernel<float><<<g2, 256, 0, stream>>>((const float*)act, offsets, (const float*)w_down, y, width, ff, n_experts);
    } else if (dtype == BLM_BF16) {
        moe_gate_up_kernel<__nv_bfloat16><<<g1, 256, 0, stream>>>((const __nv_bfloat16*)h, weights, order, offsets,
                                                                  (const __nv_bfloat16*)w_gu, (__nv_bfloat16*)act, width, ff, n_experts,
                                                                  top, scale_input);
        moe_down_kernel<__nv_bfloat16><<<g2, 256, 0, stream>>>((const __nv_bfloat16*)act, offsets, (const __nv_bfloat16*)w_down, y, width,
                                                               ff, n_experts);
    } else {
        return blm_fail(BLM_BAD_ARGUMENT, "moe_experts: dtype %d", dtype);
    }
    return blm_check_launch("moe_experts");
}

// ---------------------------------------------------------------------------------------------
// out[n] = sum_k (weight_k if the weight is on the output) y[place_of[n, k]] + extra[n]   (k in the order of the choice)
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ place_of, const float* __restrict__ weights,
                                   const T* __restrict__ extra, T* __restrict__ out, int width, int top, int scale_output) {
    const int n = blockIdx.x;
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < top; ++k) {
            const float v = y[(size_t)place_of[(size_t)n * top + k] * width + d];
            s += scale_output ? weights[(size_t)n * top + k] * v : v;
        }
        if (extra) s += to_f32(extra[(size_t)n * width + d]);
        out[(size_t)n * width + d] = from_f32<T>(s);
    }
}

BLM_API int blm_moe_combine(const float* y, const int* place_of, const float* weights, const void* extra, void* out, int dtype,
                            int n_tokens, int width, int top, int scale_output, cudaStream_t stream) {
    if (n_tokens == 0) return BLM_OK;
    BLM_REQUIRE(n_tokens > 0 && width > 0 && top > 0, "moe_combine: bad sizes");
    if (dtype == BLM_F32)
        moe_combine_kernel<float><<<n_tokens, 256, 0, stream>>>(y, place_of, weights, (const float*)extra, (float*)out, width, top, scale_output);
    else if (dtype == BLM_BF16)
        moe_combine_kernel<__nv_bfloat16><<<n_tokens, 256, 0, stream>>>(y, place_of, weights, (const __nv_bfloat16*)extra,
                                                                        (__nv_bfloat16*)out, width, top, scale_output);
    else
        return blm_fail(BLM_BAD_ARGUMENT, "moe_combine: dtype %d", dtype);
    return blm_check_launch("moe_combine");
}
