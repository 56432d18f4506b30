// Attention over a window of the latest keys plus the first keys of the sequence, with an optional sink in the
// softmax, keys and values of different sizes, and an optional gate per head.
//
//   visible(i, j) = j <= i and (i - j < window or j < keep_first)
//   p_j = exp(s_j) / (sink + sum_visible exp(s_j)),  s_j = scale q.k_j      (sink = 1: one more entry of score 0
//                                                                             that carries no value; 0: plain softmax)
//   out[n, h] = gate(n, h) * sum_j p_j v_j,  gate = sigmoid(g[n, h]) or 1
//
// The cache page of this family holds the keys [n_kv, page, dk] followed by the values [n_kv, page, dv].
// Scores, softmax and sums are fp32; q, keys and values are read in the cache's dtype.
#include "common.cuh"

BLM_API const char* blm_attention_sink_last_error() { return g_blm_error; }

// ---------------------------------------------------------------------------------------------
// After the fused projection [q | k | v | ...] (fp32 rows): the root mean square over the WHOLE q (all heads at
// once) and over the whole k, their weights, the blend of the values with an earlier layer's values of the same
// tokens, and the append of k and v to the token's place in the paged cache.
//   q_out[n, c] = q[c] / rms(q) * wq[c]            (wq == nullptr: q as it is)
//   k likewise; v <- (1 - lambda) v + lambda v_in[n] when v_in is given; v_out[n] = v when v_out is given
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void qk_norm_append_kernel(const float* __restrict__ proj, long long proj_stride, int q_cols, int k_cols, int v_cols,
                                      const float* __restrict__ wq, const float* __restrict__ wk, float eps,
                                      const float* __restrict__ lambda_p, const float* __restrict__ v_in, float* __restrict__ v_out,
                                      T* __restrict__ q_out, T* __restrict__ pool, long long page_elems, int n_kv, int dk, int dv,
                                      int page_size, const int* __restrict__ token_seq, const int* __restrict__ token_pos,
                                      const int* __restrict__ slot_of_seq, const int* __restrict__ block_table, int table_stride) {
    __shared__ float red[33];
    const int n = blockIdx.x;
    const float* p = proj + (size_t)n * proj_stride;
    float rq = 1.f, rk = 1.f;
    if (wq != nullptr) {
        float sq = 0.f, sk = 0.f;
        for (int c = threadIdx.x; c < q_cols; c += blockDim.x) sq += p[c] * p[c];
        for (int c = threadIdx.x; c < k_cols; c += blockDim.x) sk += p[q_cols + c] * p[q_cols + c];
        sq = block_sum(sq, red);
        sk = block_sum(sk, red);
        rq = 1.0f / sqrtf(sq / (float)q_cols + eps);
        rk = 1.0f / sqrtf(sk / (float)k_cols + eps);
    }
    T* qo = q_out + (size_t)n * q_cols;
    for (int c = threadIdx.x; c < q_cols; c += blockDim.x) qo[c] = from_f32<T>(wq ? p[c] * rq * wq[c] : p[c]);
    const int seq = token_seq[n];
    T* kpage = nullptr;
    T* vpage = nullptr;
    int r = 0;
    if (seq >= 0) {
        const int pos = token_pos[n];
        const int page = block_table[(size_t)slot_of_seq[seq] * table_stride + pos / page_size];
        r = pos % page_size;
        kpage = pool + (size_t)page * page_elems;
        vpage = kpage + (size_t)n_kv * page_size * dk;
    }
    if (kpage != nullptr) {
        const float* k = p + q_cols;
        for (int c = threadIdx.x; c < k_cols; c += blockDim.x) {
            const int head = c / dk, d = c % dk;
            kpage[((size_t)head * page_size + r) * dk + d] = from_f32<T>(wk ? k[c] * rk * wk[c] : k[c]);
        }
    }
    const float lambda = v_in ? lambda_p[0] : 0.f;
    const float* v = p + q_cols + k_cols;
    for (int c = threadIdx.x; c < v_cols; c += blockDim.x) {
        float x = v[c];
        if (v_in) x = (1.0f - lambda) * x + lambda * v_in[(size_t)n * v_cols + c];
        if (v_out) v_out[(size_t)n * v_cols + c] = x;
        if (vpage != nullptr) {
            const int head = c / dv, d = c % dv;
            vpage[((size_t)head * page_size + r) * dv + d] = from_f32<T>(x);
        }
    }
}

BLM_API int blm_qk_norm_append(const float* proj, long long proj_stride, int n_tokens, int n_heads, int n_kv, int dk, int dv,
                               const float* wq, const float* wk, float eps, const float* lambda_p, const float* v_in, float* v_out,
                               void* q_out, void* pool, int dtype, long long page_elems, int page_size, const int* token_seq,
                               const int* token_pos, const int* slot_of_seq, const int* block_table, int table_stride,
                               cudaStream_t stream) {
    if (n_tokens == 0) return BLM_OK;
    BLM_REQUIRE(n_tokens > 0 && n_heads > 0 && n_kv > 0 && dk > 0 && dv > 0 && page_size > 0, "qk_norm_append: bad sizes");
    BLM_REQUIRE(page_elems == (long long)n_kv * page_size * (dk + dv), "qk_norm_append: a page holds n_kv * page * (dk + dv) elements");
    BLM_REQUIRE((wq == nullptr) == (wk == nullptr), "qk_norm_append: q and k are normed together or not at all");
    BLM_REQUIRE(v_in == nullptr || lambda_p != nullptr, "qk_norm_append: blending needs its weight");
    const int q_cols = n_heads * dk, k_cols = n_kv * dk, v_cols = n_kv * dv;
    if (dtype == BLM_F32)
        qk_norm_append_kernel<float><<<n_tokens, 256, 0, stream>>>(proj, proj_stride, q_cols, k_cols, v_cols, wq, wk, eps, lambda_p, v_in,
            v_out, (float*)q_out, (float*)pool, page_elems, n_kv, dk, dv, page_size, token_seq, token_pos, slot_of_seq, block_table,
            table_stride);
    else if (dtype == BLM_BF16)
        qk_norm_append_kernel<__nv_bfloat16><<<n_tokens, 256, 0, stream>>>(proj, proj_stride, q_cols, k_cols, v_cols, wq, wk, eps, lambda_p,
            v_in, v_out, (__nv_bfloat16*)q_out, (__nv_bfloat16*)pool, page_elems, n_kv, dk, dv, page_size, token_seq, token_pos,
            slot_of_seq, block_table, table_stride);
    else
        return blm_fail(BLM_BAD_ARGUMENT, "qk_norm_append: dtype %d", dtype);
    return blm_check_launch("qk_norm_append");
}

// ---------------------------------------------------------------------------------------------
// The row kernel: one block per (query row, kv head), one warp per query head of the group (in turns when the
// group has more heads than the block has warps).  The visible keys of the row are walked in chunks of 32: the
// block stages a chunk's keys and values in shared memory, every lane of a warp scores one key, and the lanes
// then own the lanes of the output.  It serves prompts and single tokens alike.
// ---------------------------------------------------------------------------------------------
constexpr int kChunk = 32;
constexpr int kMaxVRegs = 8;      // value lanes per thread: dv <= 32 * kMaxVRegs

template <typename T>
__global__ void attention_sink_rows_kernel(const T* __restrict__ q, const T* __restrict__ pool, long long page_elems,
                                           const int* __restrict__ block_table, int table_stride, const int* __restrict__ token_seq,
                                           const int* __restrict__ token_pos, const int* __restrict__ slot_of_seq,
                                           const float* __restrict__ gate, long long gate_stride, T* __restrict__ out, int n_heads,
                                           int n_kv, int dk, int dv, int page_size, int window, int keep_first, float scale, int sink) {
    extern __shared__ float smem[];
    const int n = blockIdx.x, kvh = blockIdx.y;
    const int group = n_heads / n_kv;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int kstride = dk + 1;                        // odd row length: the lanes of a warp read one column of 32 rows
    float* ks = smem;                                  // [kChunk][dk + 1]
    float* vs = ks + kChunk * kstride;                 // [kChunk][dv]
    float* qs = vs + kChunk * dv;                      // [n_warps][dk]
    const int seq = token_seq[n];
    T* orow = out + (size_t)n * n_heads * dv;
    if (seq < 0) {                                     // a row of no sequence: zeros, nothing read
        for (int c = threadIdx.x; c < group * dv; c += blockDim.x) orow[(size_t)kvh * group * dv + c] = from_f32<T>(0.f);
        return;
    }
    const int pos = token_pos[n];
    const int* pages = block_table + (size_t)slot_of_seq[seq] * table_stride;
    const int lo = max(0, pos - window + 1);           // first key of the window
    const int n_first = min(keep_first, lo);           // kept first keys that lie before the window
    const int total = n_first + (pos - lo + 1);
    for (int h0 = 0; h0 < group; h0 += n_warps) {
        const int head = kvh * group + h0 + warp;
        const bool active = h0 + warp < group;
        __syncthreads();                               // the chunk buffers and qs of the heads before are done with
        if (active)
            for (int d = lane; d < dk; d += 32) qs[warp * dk + d] = to_f32(q[((size_t)n * n_heads + head) * dk + d]);
        float m = sink ? 0.f : -INFINITY, l = sink ? 1.f : 0.f;
        float acc[kMaxVRegs];
#pragma unroll
        for (int i = 0; i < kMaxVRegs; ++i) acc[i] = 0.f;
        for (int c0 = 0; c0 < total; c0 += kChunk) {
            __syncthreads();
            for (int idx = threadIdx.x; idx < kChunk * dk; idx += blockDim.x) {
                const int row = idx / dk, d = idx % dk, i = c0 + row;
                float v = 0.f;
                if (i < total) {
                    const int j = i < n_first ? i : lo + (i - n_first);
                    const T* kpage = pool + (size_t)pages[j / page_size] * page_elems;
                    v = to_f32(kpage[((size_t)kvh * page_size + j % page_size) * dk + d]);
                }
                ks[row * kstride + d] = v;
            }
            for (int idx = threadIdx.x; idx < kChunk * dv; idx += blockDim.x) {
                const int row = idx / dv, d = idx % dv, i = c0 + row;
                float v = 0.f;
                if (i < total) {
                    const int j = i < n_first ? i : lo + (i - n_first);
                    const T* vpage = pool + (size_t)pages[j / page_size] * page_elems + (size_t)n_kv * page_size * dk;
                    v = to_f32(vpage[((size_t)kvh * page_size + j % page_size) * dv + d]);
                }
                vs[row * dv + d] = v;
            }
            __syncthreads();
            if (active) {
                float s = -INFINITY;
                if (c0 + lane < total) {
                    float dot = 0.f;
                    const float* kr = ks + lane * kstride;
                    const float* qr = qs + warp * dk;
                    for (int d = 0; d < dk; ++d) dot = fmaf(qr[d], kr[d], dot);
                    s = dot * scale;
                }
                const float m_new = fmaxf(m, warp_max(s));
                const float p = (c0 + lane < total) ? expf(s - m_new) : 0.f;
                const float corr = expf(m - m_new);          // m = -inf only before the first chunk, where m_new is finite
                l = l * corr + warp_sum(p);
                m = m_new;
#pragma unroll
                for (int i = 0; i < kMaxVRegs; ++i) acc[i] *= corr;
                const int rows = min(kChunk, total - c0);
                for (int j = 0; j < rows; ++j) {
                    const float pj = __shfl_sync(0xffffffffu, p, j);
#pragma unroll
                    for (int i = 0; i < kMaxVRegs; ++i) {
                        const int d = lane + 32 * i;
                        if (d < dv) acc[i] = fmaf(pj, vs[j * dv + d], acc[i]);
                    }
                }
            }
        }
        if (active) {
            float g = 1.f;
            if (gate != nullptr) g = 1.0f / (1.0f + expf(-gate[(size_t)n * gate_stride + head]));
            const float inv = l > 0.f ? g / l : 0.f;
#pragma unroll
            for (int i = 0; i < kMaxVRegs; ++i) {
                const int d = lane + 32 * i;
                if (d < dv) orow[(size_t)head * dv + d] = from_f32<T>(acc[i] * inv);
            }
        }
    }
}

template <typename T>
static int launch_rows(const void* q, const void* pool, long long page_elems, const int* block_table, int table_stride,
                       const int* token_seq, const int* token_pos, const int* slot_of_seq, const float* gate, long long gate_stride,
                       void* out, int n_tokens, int n_heads, int n_kv, int dk, int dv, int page_size, int window, int keep_first,
                       float scale, int sink, cudaStream_t stream) {
    const int group = n_heads / n_kv;
    const int warps = group < 8 ? group : 8;
    const size_t smem = ((size_t)kChunk * (dk + 1) + (size_t)kChunk * dv + (size_t)warps * dk) * sizeof(float);
    if (smem > 48 * 1024) {
        BLM_REQUIRE(smem <= 200 * 1024, "attention_sink: heads of %d and %d lanes need %zu bytes of shared memory", dk, dv, smem);
        cudaError_t e = cudaFuncSetAttribute(attention_sink_rows_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "attention_sink: %s", cudaGetErrorString(e));
    }
    attention_sink_rows_kernel<T><<<dim3(n_tokens, n_kv), warps * 32, smem, stream>>>(
        (const T*)q, (const T*)pool, page_elems, block_table, table_stride, token_seq, token_pos, slot_of_seq, gate, gate_stride,
        (T*)out, n_heads, n_kv, dk, dv, page_size, window, keep_first, scale, sink);
    return blm_check_launch("attention_sink");
}

BLM_API int blm_attention_sink(const void* q, const void* pool, int dtype, long long page_elems, const int* block_table,
                               int table_stride, const int* token_seq, const int* token_pos, const int* slot_of_seq,
                               const float* gate, long long gate_stride, void* out, int n_tokens, int n_heads, int n_kv, int dk,
                               int dv, int page_size, int window, int keep_first, float scale, int sink, cudaStream_t stream) {
    if (n_tokens == 0) return BLM_OK;
    BLM_REQUIRE(n_tokens > 0 && n_heads > 0 && n_kv > 0 && n_heads % n_kv == 0 && dk > 0 && dv > 0 && page_size > 0,
                "attention_sink: bad sizes");
    BLM_REQUIRE(dv <= 32 * kMaxVRegs, "attention_sink: values of %d lanes; at most %d", dv, 32 * kMaxVRegs);
    BLM_REQUIRE(window >= 1 && keep_first >= 0, "attention_sink: window %d, kept first %d", window, keep_first);
    BLM_REQUIRE(page_elems == (long long)n_kv * page_size * (dk + dv), "attention_sink: a page holds n_kv * page * (dk + dv) elements");
    BLM_REQUIRE(n_kv <= 65535, "attention_sink: %d kv heads", n_kv);
    if (dtype == BLM_F32)
        return launch_rows<float>(q, pool, page_elems, block_table, table_stride, token_seq, token_pos, slot_of_seq, gate, gate_stride,
                                  out, n_tokens, n_heads, n_kv, dk, dv, page_size, window, keep_first, scale, sink, stream);
    if (dtype == BLM_BF16)
        return launch_rows<__nv_bfloat16>(q, pool, page_elems, block_table, table_stride, token_seq, token_pos, slot_of_seq, gate,
                                          gate_stride, out, n_tokens, n_heads, n_kv, dk, dv, page_size, window, keep_first, scale, sink,
                                          stream);
    return blm_fail(BLM_BAD_ARGUMENT, "attention_sink: dtype %d", dtype);
}
