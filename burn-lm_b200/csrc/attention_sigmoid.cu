// Causal attention without a softmax, with the heads' weights mixed before they meet the values:
//     s_h(i, j) = scale q_hi . k_cj (c the key/value head of h), optionally capped: cap tanh(s / cap)
//     w_h(i, j) = sigmoid(s_h(i, j) + bias_h) for j <= i, else 0          (not normalised over the keys)
//     m_h(i, j) = sum_g talk[h, g] w_g(i, j)                              (talk null: m = w)
//     out_h(i)  = sum_j m_h(i, j) v_cj
// and the kernel in front of it: projection bias, rotation of the first `rot` lanes of every q and k head (lane i
// with lane i + rot / 2, angle = position * freq[i], taken in fp64 and applied in fp32), append of k and v to the paged cache.
// Scores, weights, the mix and the sums over keys are fp32 in both dtypes.
//
// Because nothing normalises over the keys, a query's keys can be cut into ranges whose partial outputs simply add:
// grid.y blocks take a range each and a second kernel adds the ranges in order.  A block owns BQ query rows of one
// sequence with ALL heads (the mix needs every head's weight at a key), walks its keys a chunk of a cache page at a
// time: scores of all heads, mix, then the values; outputs are kept in registers.
#include "common.cuh"

BLM_API const char* blm_attention_sigmoid_last_error() { return g_blm_error; }

constexpr int kThreads = 256;

// ---------------------------------------------------------------------------------------------
// bias + rotation + append
//   proj fp32 [N, stride]: q heads (H x dk), k heads (G x dk), v heads (G x dv); bias [that width] or null
//   q_out [N, H dk]; a cache page: keys [G][page][dk] then values [G][page][dv]
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void bias_rope_append_kernel(const float* __restrict__ proj, long long stride, const float* __restrict__ bias,
                                        const double* __restrict__ freq, int rot, T* __restrict__ q_out, T* __restrict__ pool,
                                        const int* __restrict__ token_seq, const int* __restrict__ token_pos,
                                        const int* __restrict__ slot_of_seq, const int* __restrict__ block_table, int table_stride,
                                        int H, int G, int dk, int dv, int page) {
    const int n = blockIdx.y;
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    const int qk = (H + G) * dk;
    const int width = qk + G * dv;
    if (e >= width) return;
    const float* row = proj + (size_t)n * stride;
    const int pos = token_pos[n];
    float val = row[e] + (bias ? bias[e] : 0.f);
    int head = 0, lane = 0;
    if (e < qk) {
        head = e / dk;
        lane = e % dk;
        if (lane < rot) {
            const int half = rot >> 1;
            const int i = lane < half ? lane : lane - half;
            const int pe = lane < half ? e + half : e - half;
            const float other = row[pe] + (bias ? bias[pe] : 0.f);
            double sd, cd;
            sincos((double)pos * freq[i], &sd, &cd);     // the angle and its sine and cosine in fp64, applied in fp32
            const float s = (float)sd, c = (float)cd;
            val = lane < half ? val * c - other * s : val * c + other * s;
        }
        if (head < H) {
            q_out[(size_t)n * H * dk + e] = from_f32<T>(val);
            return;
        }
        head -= H;
    } else {
        head = (e - qk) / dv;
        lane = (e - qk) % dv;
    }
    const int seq = token_seq[n];
    if (seq < 0) return;             // a row of no sequence: nothing of it reaches the cache
    const int pg = block_table[(size_t)slot_of_seq[seq] * table_stride + pos / page];
    T* base = pool + (size_t)pg * G * page * (dk + dv);
    const int at = pos % page;
    if (e < qk) base[((size_t)head * page + at) * dk + lane] = from_f32<T>(val);
    else base[(size_t)G * page * dk + ((size_t)head * page + at) * dv + lane] = from_f32<T>(val);
}

BLM_API int blm_bias_rope_append(const float* proj, long long stride, const float* bias, const double* freq, int rot, void* q_out,
                                 void* pool, int dtype, const int* token_seq, const int* token_pos, const int* slot_of_seq,
                                 const int* block_table, int table_stride, int n, int H, int G, int dk, int dv, int page,
                                 cudaStream_t stream) {
    if (n == 0) return BLM_OK;
    BLM_REQUIRE(H > 0 && G > 0 && dk > 0 && dv > 0 && page > 0, "bias_rope_append: bad sizes");
    BLM_REQUIRE(rot >= 0 && rot <= dk && rot % 2 == 0 && (rot == 0 || freq != nullptr), "bias_rope_append: %d rotated lanes of %d", rot, dk);
    BLM_REQUIRE(n <= 65535, "bias_rope_append: a step of %d rows; this kernel takes 65,535", n);
    const int width = (H + G) * dk + G * dv;
    dim3 grid((width + 255) / 256, n);
    if (dtype == BLM_F32)
        bias_rope_append_kernel<float><<<grid, 256, 0, stream>>>(proj, stride, bias, freq, rot, (float*)q_out, (float*)pool, token_seq,
                                                                 token_pos, slot_of_seq, block_table, table_stride, H, G, dk, dv, page);
    else if (dtype == BLM_BF16)
        bias_rope_append_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(proj, stride, bias, freq, rot, (__nv_bfloat16*)q_out,
                                                                         (__nv_bfloat16*)pool, token_seq, token_pos, slot_of_seq,
                                                                         block_table, table_stride, H, G, dk, dv, page);
    else
        return blm_fail(BLM_BAD_ARGUMENT, "bias_rope_append: dtype %d", dtype);
    return blm_check_launch("bias_rope_append");
}

// ---------------------------------------------------------------------------------------------
// the attention
// ---------------------------------------------------------------------------------------------
template <typename T> struct Vec;
template <> struct Vec<float> { static constexpr int n = 4; };
template <> struct Vec<__nv_bfloat16> { static constexpr int n = 8; };

// rows are padded to a multiple of a 16-byte vector, plus one vector so that rows start in different banks
template <typename T> __host__ __device__ inline int padded(int d) { return (d + Vec<T>::n - 1) / Vec<T>::n * Vec<T>::n + Vec<T>::n; }

__device__ __forceinline__ float dot16(const float* a, const float* b, int n) {
    float acc = 0.f;
    for (int i = 0; i < n; i += 4) {
        const float4 x = *reinterpret_cast<const float4*>(a + i), y = *reinterpret_cast<const float4*>(b + i);
        acc += x.x * y.x;
        acc += x.y * y.y;
        acc += x.z * y.z;
        acc += x.w * y.w;
    }
    return acc;
}
__device__ __forceinline__ float dot16(const __nv_bfloat16* a, const __nv_bfloat16* b, int n) {
    float acc = 0.f;
    for (int i = 0; i < n; i += 8) {
        const uint4 x = *reinterpret_cast<const uint4*>(a + i), y = *reinterpret_cast<const uint4*>(b + i);
        const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&x);
        const __nv_bfloat162* yp = reinterpret_cast<const __nv_bfloat162*>(&y);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(xp[e]), g = __bfloat1622float2(yp[e]);
            acc += f.x * g.x;
            acc += f.y * g.y;
        }
    }
    return acc;
}

// One row of `d` elements from global to shared memory, its lanes up to `dp` zeroed, by the lanes of a warp: in 16-byte
// pieces when the row allows (d a multiple of a piece, both ends aligned), else element by element.  `live` false: zeros.
template <typename T>
__device__ __forceinline__ void stage_row(T* dst, const T* src, int d, int dp, bool live, int lane) {
    constexpr int V = Vec<T>::n;
    if (d % V == 0 && (((size_t)src | (size_t)dst) & 15) == 0) {
        for (int c = lane; c < dp / V; c += 32) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (live && c < d / V) v = *reinterpret_cast<const uint4*>(src + c * V);
            *reinterpret_cast<uint4*>(dst + c * V) = v;
        }
    } else {
        for (int c = lane; c < dp; c += 32) dst[c] = (live && c < d) ? src[c] : from_f32<T>(0.f);
    }
}

struct SigmoidAttnArgs {
    const void* q;            // [N, H dk]
    const void* pool;         // pages: keys [G][page][dk] then values [G][page][dv]
    const int* block_table;
    int table_stride;
    const int* cu_seqlens;
    const int* slot_of_seq;
    const int* start_pos;
    const float* talk;        // [H, H] or null
    const float* head_bias;   // [H] or null
    void* out;                // [N, H dv] in the activation dtype (one range)
    float* partial;           // [ranges][N][H dv] fp32 (several ranges)
    int n_tokens, n_seqs, q_tiles, H, G, dk, dv, page, BQ, KC, ranges;
    float scale, softcap;
};

template <typename T, int ACC>
__global__ void __launch_bounds__(kThreads) sigmoid_attn_kernel(const SigmoidAttnArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int H = a.H, G = a.G, dk = a.dk, dv = a.dv, BQ = a.BQ, KC = a.KC;
    const int dkp = padded<T>(dk), dvp = padded<T>(dv);
    float* Ts = reinterpret_cast<float*>(smem_raw);                 // [H][H]
    float* pbs = Ts + (H * H + 3) / 4 * 4;                           // [H]
    float* Ss = pbs + ((H + 3) / 4) * 4;                             // [H][BQ][KC]
    float* Ms = Ss + H * BQ * KC;                                    // [H][BQ][KC]
    T* Qs = reinterpret_cast<T*>(Ms + H * BQ * KC);                  // [H][BQ][dkp]
    T* KVs = Qs + (size_t)H * BQ * dkp;                              // [G][KC][kvp]
    const int tid = threadIdx.x;
    const int seq = blockIdx.x / a.q_tiles, tile = a.q_tiles - 1 - blockIdx.x % a.q_tiles;     // a sequence's last rows, with the most keys, first
    const int first = a.cu_seqlens[seq];
    const int n_new = a.cu_seqlens[seq + 1] - first;
    const int i0 = tile * BQ;
    if (i0 >= n_new) return;
    const int nq = min(BQ, n_new - i0);
    const int start = a.start_pos[seq];
    const int kv_hi = start + i0 + nq;                  // keys 0 .. kv_hi - 1 are seen by some row of the tile
    const int chunks = (kv_hi + KC - 1) / KC;
    const int per = (chunks + a.ranges - 1) / a.ranges;
    const int c_lo = blockIdx.y * per, c_hi = min(chunks, c_lo + per);
    const int* table = a.block_table + (size_t)a.slot_of_seq[seq] * a.table_stride;
    const int per_kv = H / G;
    const int HD = H * dv;

    for (int e = tid; e < H * H; e += kThreads) Ts[e] = a.talk ? a.talk[e] : (e / H == e % H ? 1.f : 0.f);
    for (int e = tid; e < H; e += kThreads) pbs[e] = a.head_bias ? a.head_bias[e] : 0.f;
    // the tile's queries, rows beyond the tile and lanes beyond dk as zeros
    const T* q = reinterpret_cast<const T*>(a.q);
    const int lane = tid & 31, warp = tid >> 5;
    for (int r = warp; r < H * BQ; r += kThreads / 32) {           // a warp a row
        const int i = r % BQ, h = r / BQ;
        stage_row(Qs + (size_t)r * dkp, q + (size_t)(first + i0 + i) * H * dk + h * dk, dk, dkp, i < nq, lane);
    }
    float acc[ACC];
#pragma unroll
    for (int x = 0; x < ACC; ++x) acc[x] = 0.f;
    const int n_out = H * BQ * dv;                       // output e = (h, i, p), p fastest; thread tid owns e = tid + x * kThreads
    const T* pool = reinterpret_cast<const T*>(a.pool);
    const size_t page_elems = (size_t)G * a.page * (dk + dv);
    const bool cap = a.softcap > 0.f;
    const float inv_cap = cap ? 1.0f / a.softcap : 0.f;

    for (int ch = c_lo; ch < c_hi; ++ch) {
        const int j0 = ch * KC;
        const T* pg = pool + (size_t)table[j0 / a.page] * page_elems;
        const int at0 = j0 % a.page;
        __syncthreads();                                  // the chunk before is done with KVs, Ss and Ms
        for (int r = warp; r < G * KC; r += kThreads / 32) {
            const int j = r % KC, g = r / KC;
            stage_row(KVs + (size_t)r * dkp, pg + ((size_t)g * a.page + at0 + j) * dk, dk, dkp, j0 + j < kv_hi, lane);
        }
        __syncthreads();
        // scores and weights of all heads
        for (int e = tid; e < H * BQ * KC; e += kThreads) {
            const int j = e % KC, i = (e / KC) % BQ, h = e / (KC * BQ);
            float w = 0.f;
            if (i < nq && j0 + j <= start + i0 + i) {
                float s = dot16(Qs + (size_t)(h * BQ + i) * dkp, KVs + (size_t)((h / per_kv) * KC + j) * dkp, dkp - Vec<T>::n) * a.scale;
                if (cap) s = a.softcap * tanhf(s * inv_cap);
                w = 1.0f / (1.0f + expf(-(s + pbs[h])));
            }
            Ss[e] = w;
        }
        __syncthreads();
        // the values take the keys' place while the weights are mixed
        for (int r = warp; r < G * KC; r += kThreads / 32) {
            const int j = r % KC, g = r / KC;
            stage_row(KVs + (size_t)r * dvp, pg + (size_t)G * a.page * dk + ((size_t)g * a.page + at0 + j) * dv, dv, dvp, j0 + j < kv_hi, lane);
        }
        const int ij = BQ * KC;
        for (int e = tid; e < H * ij; e += kThreads) {
            const int x = e % ij, h = e / ij;
            const float* t = Ts + h * H;
            float m = 0.f;
            for (int g = 0; g < H; ++g) m += t[g] * Ss[g * ij + x];
            Ms[e] = m;
        }
        __syncthreads();
#pragma unroll
        for (int x = 0; x < ACC; ++x) {
            const int e = tid + x * kThreads;
            if (e < n_out) {
                const int p = e % dv, i = (e / dv) % BQ, h = e / (dv * BQ);
                const float* m = Ms + (size_t)(h * BQ + i) * KC;
                const T* v = KVs + (size_t)((h / per_kv) * KC) * dvp + p;
                float s = acc[x];
                for (int j = 0; j < KC; ++j) s += m[j] * to_f32(v[(size_t)j * dvp]);
                acc[x] = s;
            }
        }
    }
#pragma unroll
    for (int x = 0; x < ACC; ++x) {
        const int e = tid + x * kThreads;
        if (e < n_out) {
            const int p = e % dv, i = (e / dv) % BQ, h = e / (dv * BQ);
            if (i < nq) {
                const size_t at = (size_t)(first + i0 + i) * HD + h * dv + p;
                if (a.ranges > 1) a.partial[(size_t)blockIdx.y * a.n_tokens * HD + at] = acc[x];
                else reinterpret_cast<T*>(a.out)[at] = from_f32<T>(acc[x]);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// The same attention on the tensor cores (bfloat16): 16 query rows of one sequence a block, all heads' scores by
// mma.sync m16n8k16 (Q rows x a chunk of keys), the weights and their mix in fp32 on the CUDA cores, the mixed weights
// rounded to bfloat16 for the second product with the values.  Heads are cut into grid.z groups for the second product
// only (every block needs every head's weights for the mix), so that a block's outputs fit its registers.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void ldsm_x4(unsigned (&r)[4], const void* p) {
    const unsigned addr = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2(unsigned (&r)[2], const void* p) {
    const unsigned addr = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2_trans(unsigned (&r)[2], const void* p) {
    const unsigned addr = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const unsigned (&a)[4], const unsigned (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

constexpr int kRows = 16;          // query rows of a block of the tensor-core kernel
constexpr int kMmaMinRows = 2;      // steps whose longest run is one token run the kernel whose rows are heads, or the CUDA-core kernel
constexpr int kThreadsMma = 512;   // sixteen warps: the weights' exponentials and the mix want many warps in flight

struct MmaLayout {                 // strides and offsets (bytes) of the block's shared memory
    int dkp, dvp, kvp, ssp, msp, hown, hpad;
    size_t ts, pbs, ss, ms, qs, kv, total;
};

__host__ __device__ inline MmaLayout mma_layout(int H, int G, int dk, int dv, int KC, int HG) {
    MmaLayout l;
    l.dkp = dk + 8;
    l.dvp = dv + 8;
    l.kvp = l.dkp > l.dvp ? l.dkp : l.dvp;
    l.ssp = KC + 8;                                     // floats a row of weights
    l.msp = KC + 8;                                     // bfloat16 a row of mixed weights
    l.hown = H / HG;
    l.hpad = (l.hown + 7) / 8 * 8;
    l.ts = 0;                                           // [H][hpad] floats: talk transposed, own heads by columns
    l.pbs = l.ts + (size_t)H * l.hpad * 4;              // [H] floats
    l.ss = l.pbs + (size_t)((H + 3) / 4 * 4) * 4;       // [H][16][ssp] floats
    l.ms = l.ss + (size_t)H * kRows * l.ssp * 4;        // [hown][16][msp] bfloat16
    l.qs = l.ms + (size_t)l.hown * kRows * l.msp * 2;   // [H][16][dkp] bfloat16
    l.kv = l.qs + (size_t)H * kRows * l.dkp * 2;        // [G][KC][kvp] bfloat16
    l.total = l.kv + (size_t)G * KC * l.kvp * 2;
    return l;
}

template <int NT>      // 16 x 8 output tiles a warp owns
__global__ void __launch_bounds__(kThreadsMma) sigmoid_attn_mma_kernel(const SigmoidAttnArgs a, int HG) {
    typedef __nv_bfloat16 T;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int H = a.H, G = a.G, dk = a.dk, dv = a.dv, KC = a.KC;
    const MmaLayout L = mma_layout(H, G, dk, dv, KC, HG);
    float* Ts = reinterpret_cast<float*>(smem_raw + L.ts);
    float* pbs = reinterpret_cast<float*>(smem_raw + L.pbs);
    float* Ss = reinterpret_cast<float*>(smem_raw + L.ss);
    T* Ms = reinterpret_cast<T*>(smem_raw + L.ms);
    T* Qs = reinterpret_cast<T*>(smem_raw + L.qs);
    T* KVs = reinterpret_cast<T*>(smem_raw + L.kv);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int seq = blockIdx.x / a.q_tiles, tile = a.q_tiles - 1 - blockIdx.x % a.q_tiles;     // a sequence's last rows, with the most keys, first
    const int first = a.cu_seqlens[seq];
    const int n_new = a.cu_seqlens[seq + 1] - first;
    const int i0 = tile * kRows;
    if (i0 >= n_new) return;
    const int nq = min(kRows, n_new - i0);
    const int start = a.start_pos[seq];
    const int kv_hi = start + i0 + nq;
    const int chunks = (kv_hi + KC - 1) / KC;
    const int per = (chunks + a.ranges - 1) / a.ranges;
    const int c_lo = blockIdx.y * per, c_hi = min(chunks, c_lo + per);
    const int* table = a.block_table + (size_t)a.slot_of_seq[seq] * a.table_stride;
    const int per_kv = H / G;
    const int HD = H * dv;
    const int h0 = blockIdx.z * L.hown;                 // this block's heads for the second product
    const int dv8 = dv / 8;
    const int own_tiles = L.hown * dv8;
    const int g_lo = h0 / per_kv, g_n = (h0 + L.hown - 1) / per_kv - g_lo + 1;

    for (int e = tid; e < H * L.hpad; e += kThreadsMma) {
        const int g = e / L.hpad, hl = e % L.hpad;
        Ts[e] = hl < L.hown ? (a.talk ? a.talk[(size_t)(h0 + hl) * H + g] : (h0 + hl == g ? 1.f : 0.f)) : 0.f;
    }
    for (int e = tid; e < H; e += kThreadsMma) pbs[e] = a.head_bias ? a.head_bias[e] : 0.f;
    const T* q = reinterpret_cast<const T*>(a.q);
    const int dk8 = dk / 8;
    for (int e = tid; e < H * kRows * dk8; e += kThreadsMma) {          // 16-byte pieces of the tile's queries
        const int c = e % dk8, i = (e / dk8) % kRows, h = e / (dk8 * kRows);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (i < nq) v = *reinterpret_cast<const uint4*>(q + (size_t)(first + i0 + i) * H * dk + h * dk + c * 8);
        *reinterpret_cast<uint4*>(Qs + (size_t)(h * kRows + i) * L.dkp + c * 8) = v;
    }
    float acc[NT][4];
#pragma unroll
    for (int x = 0; x < NT; ++x) acc[x][0] = acc[x][1] = acc[x][2] = acc[x][3] = 0.f;
    const T* pool = reinterpret_cast<const T*>(a.pool);
    const size_t page_elems = (size_t)G * a.page * (dk + dv);
    const bool cap = a.softcap > 0.f;
    const float inv_cap = cap ? 1.0f / a.softcap : 0.f;
    const int n_tiles_s = H * (KC / 8);                  // score tiles of a chunk: (head, 8 keys)

    for (int ch = c_lo; ch < c_hi; ++ch) {
        const int j0 = ch * KC;
        const T* pg = pool + (size_t)table[j0 / a.page] * page_elems;
        const int at0 = j0 % a.page;
        __syncthreads();
        for (int e = tid; e < G * KC * dk8; e += kThreadsMma) {
            const int c = e % dk8, j = (e / dk8) % KC, g = e / (dk8 * KC);
            uint4 v = make_uint4(0, 0, 0, 0);
            if (j0 + j < kv_hi) v = *reinterpret_cast<const uint4*>(pg + ((size_t)g * a.page + at0 + j) * dk + c * 8);
            *reinterpret_cast<uint4*>(KVs + (size_t)(g * KC + j) * L.dkp + c * 8) = v;
        }
        __syncthreads();
        // scores of all heads on the tensor cores, weights in fp32
        for (int s = warp; s < n_tiles_s; s += kThreadsMma / 32) {
            const int h = s / (KC / 8), nt = s % (KC / 8);
            float c4[4] = {0.f, 0.f, 0.f, 0.f};
            const T* qa = Qs + (size_t)(h * kRows + (lane & 15)) * L.dkp + (lane >> 4) * 8;
            const T* kb = KVs + (size_t)((h / per_kv) * KC + nt * 8 + (lane & 7)) * L.dkp + ((lane >> 3) & 1) * 8;
            for (int kk = 0; kk < dk; kk += 16) {
                unsigned af[4], bf[2];
                ldsm_x4(af, qa + kk);
                ldsm_x2(bf, kb + kk);
                mma_16816(c4, af, bf);
            }
            const float pb = pbs[h];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int i = (lane >> 2) + 8 * r;
                float w2[2];
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    const int j = nt * 8 + 2 * (lane & 3) + cc;
                    float w = 0.f;
                    if (i < nq && j0 + j <= start + i0 + i) {
                        float sc = c4[2 * r + cc] * a.scale;
                        if (cap) sc = a.softcap * (1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * sc * inv_cap)));     // cap tanh(sc / cap)
                        w = __fdividef(1.0f, 1.0f + __expf(-(sc + pb)));
                    }
                    w2[cc] = w;
                }
                *reinterpret_cast<float2*>(Ss + (size_t)(h * kRows + i) * L.ssp + nt * 8 + 2 * (lane & 3)) = make_float2(w2[0], w2[1]);
            }
        }
        __syncthreads();
        // the values take the keys' place while the weights of this block's heads are mixed
        for (int e = tid; e < g_n * KC * dv8; e += kThreadsMma) {          // only the value heads this block's heads read
            const int c = e % dv8, j = (e / dv8) % KC, g = g_lo + e / (dv8 * KC);
            uint4 v = make_uint4(0, 0, 0, 0);
            if (j0 + j < kv_hi) v = *reinterpret_cast<const uint4*>(pg + (size_t)G * a.page * dk + ((size_t)g * a.page + at0 + j) * dv + c * 8);
            *reinterpret_cast<uint4*>(KVs + (size_t)(g * KC + j) * L.dvp + c * 8) = v;
        }
        for (int e = tid; e < (L.hpad / 8) * kRows * KC; e += kThreadsMma) {
            const int j = e % KC, i = (e / KC) % kRows, hc = e / (KC * kRows);
            float m[8];
#pragma unroll
            for (int x = 0; x < 8; ++x) m[x] = 0.f;
            const float* sp = Ss + (size_t)i * L.ssp + j;
            const float* tp = Ts + hc * 8;
            for (int g = 0; g < (i < nq ? H : 0); ++g) {      // rows beyond the tile's queries (single tokens) stay zero
                const float sv = sp[(size_t)g * kRows * L.ssp];
                const float4 t0 = *reinterpret_cast<const float4*>(tp + (size_t)g * L.hpad);
                const float4 t1 = *reinterpret_cast<const float4*>(tp + (size_t)g * L.hpad + 4);
                m[0] += t0.x * sv; m[1] += t0.y * sv; m[2] += t0.z * sv; m[3] += t0.w * sv;
                m[4] += t1.x * sv; m[5] += t1.y * sv; m[6] += t1.z * sv; m[7] += t1.w * sv;
            }
#pragma unroll
            for (int x = 0; x < 8; ++x)
                if (hc * 8 + x < L.hown) Ms[(size_t)((hc * 8 + x) * kRows + i) * L.msp + j] = __float2bfloat16_rn(m[x]);
        }
        __syncthreads();
        // mixed weights x values
#pragma unroll
        for (int x = 0; x < NT; ++x) {
            const int t = warp * NT + x;
            if (t < own_tiles) {
                const int hl = t / dv8, nt = t % dv8;
                const T* ma = Ms + (size_t)(hl * kRows + (lane & 15)) * L.msp + (lane >> 4) * 8;
                const T* vb = KVs + (size_t)(((h0 + hl) / per_kv) * KC + (lane & 15)) * L.dvp + nt * 8;
                for (int kk = 0; kk < KC; kk += 16) {
                    unsigned af[4], bf[2];
                    ldsm_x4(af, ma + kk);
                    ldsm_x2_trans(bf, vb + (size_t)kk * L.dvp);
                    mma_16816(acc[x], af, bf);
                }
            }
        }
    }
#pragma unroll
    for (int x = 0; x < NT; ++x) {
        const int t = warp * NT + x;
        if (t < own_tiles) {
            const int hl = t / dv8, nt = t % dv8;
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int i = (lane >> 2) + 8 * r;
                if (i < nq) {
                    const size_t at = (size_t)(first + i0 + i) * HD + (h0 + hl) * dv + nt * 8 + 2 * (lane & 3);
                    if (a.ranges > 1) {
                        *reinterpret_cast<float2*>(a.partial + (size_t)blockIdx.y * a.n_tokens * HD + at) = make_float2(acc[x][2 * r], acc[x][2 * r + 1]);
                    } else {
                        *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<T*>(a.out) + at) = __floats2bfloat162_rn(acc[x][2 * r], acc[x][2 * r + 1]);
                    }
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Single tokens on the tensor cores (bfloat16): one query a sequence, so the rows of a tile are the HEADS of a key/value
// head (up to 16), as in the dense decoder's decode kernel.  A block owns (sequence, range of keys) with all heads: per
// chunk of keys one score tile per key/value head, the weights of all heads in fp32, the mix, one value product per
// key/value head.  No head groups: a block's outputs are heads x value lanes.
// ---------------------------------------------------------------------------------------------
struct RowsLayout {
    int dkp, dvp, kvp, ssp, msp, hpad;
    size_t ts, pbs, ss, ms, qs, kv, total;
};

__host__ __device__ inline RowsLayout rows_layout(int H, int G, int dk, int dv, int KC) {
    RowsLayout l;
    l.dkp = dk + 8;
    l.dvp = dv + 8;
    l.kvp = l.dkp > l.dvp ? l.dkp : l.dvp;
    l.ssp = KC;
    l.msp = KC + 8;
    l.hpad = (H + 7) / 8 * 8;
    l.ts = 0;                                               // [H][hpad] floats: talk transposed
    l.pbs = l.ts + (size_t)H * l.hpad * 4;                  // [H] floats
    l.ss = l.pbs + (size_t)((H + 3) / 4 * 4) * 4;           // [H][ssp] floats: the one query's weights
    l.ms = l.ss + (size_t)H * l.ssp * 4;                    // [G][16][msp] bfloat16: mixed weights, a head a row
    l.qs = l.ms + (size_t)G * kRows * l.msp * 2;            // [G][16][dkp] bfloat16: the query, a head a row
    l.kv = l.qs + (size_t)G * kRows * l.dkp * 2;            // [G][KC][kvp] bfloat16
    l.total = l.kv + (size_t)G * KC * l.kvp * 2;
    return l;
}

template <int NT>
__global__ void __launch_bounds__(kThreads) sigmoid_attn_rows_kernel(const SigmoidAttnArgs a) {
    typedef __nv_bfloat16 T;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int H = a.H, G = a.G, dk = a.dk, dv = a.dv, KC = a.KC;
    const RowsLayout L = rows_layout(H, G, dk, dv, KC);
    float* Ts = reinterpret_cast<float*>(smem_raw + L.ts);
    float* pbs = reinterpret_cast<float*>(smem_raw + L.pbs);
    float* Ss = reinterpret_cast<float*>(smem_raw + L.ss);
    T* Ms = reinterpret_cast<T*>(smem_raw + L.ms);
    T* Qs = reinterpret_cast<T*>(smem_raw + L.qs);
    T* KVs = reinterpret_cast<T*>(smem_raw + L.kv);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int seq = blockIdx.x;
    const int first = a.cu_seqlens[seq];
    if (a.cu_seqlens[seq + 1] - first != 1) return;      // this kernel serves sequences that bring one token
    const int kv_hi = a.start_pos[seq] + 1;
    const int chunks = (kv_hi + KC - 1) / KC;
    const int per = (chunks + a.ranges - 1) / a.ranges;
    const int c_lo = blockIdx.y * per, c_hi = min(chunks, c_lo + per);
    const int* table = a.block_table + (size_t)a.slot_of_seq[seq] * a.table_stride;
    const int per_kv = H / G;
    const int HD = H * dv;
    const int dk8 = dk / 8, dv8 = dv / 8;
    const int own_tiles = G * dv8;

    for (int e = tid; e < H * L.hpad; e += kThreads) {
        const int g = e / L.hpad, h = e % L.hpad;
        Ts[e] = h < H ? (a.talk ? a.talk[(size_t)h * H + g] : (h == g ? 1.f : 0.f)) : 0.f;
    }
    for (int e = tid; e < H; e += kThreads) pbs[e] = a.head_bias ? a.head_bias[e] : 0.f;
    for (int e = tid; e < G * kRows * L.msp / 8; e += kThreads) reinterpret_cast<uint4*>(Ms)[e] = make_uint4(0, 0, 0, 0);
    const T* q = reinterpret_cast<const T*>(a.q) + (size_t)first * H * dk;
    for (int e = tid; e < G * kRows * dk8; e += kThreads) {
        const int c = e % dk8, r = (e / dk8) % kRows, g = e / (dk8 * kRows);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < per_kv) v = *reinterpret_cast<const uint4*>(q + (size_t)(g * per_kv + r) * dk + c * 8);
        *reinterpret_cast<uint4*>(Qs + (size_t)(g * kRows + r) * L.dkp + c * 8) = v;
    }
    float acc[NT][4];
#pragma unroll
    for (int x = 0; x < NT; ++x) acc[x][0] = acc[x][1] = acc[x][2] = acc[x][3] = 0.f;
    const T* pool = reinterpret_cast<const T*>(a.pool);
    const size_t page_elems = (size_t)G * a.page * (dk + dv);
    const bool cap = a.softcap > 0.f;
    const float inv_cap = cap ? 1.0f / a.softcap : 0.f;
    const int kc8 = KC / 8;

    for (int ch = c_lo; ch < c_hi; ++ch) {
        const int j0 = ch * KC;
        const T* pg = pool + (size_t)table[j0 / a.page] * page_elems;
        const int at0 = j0 % a.page;
        __syncthreads();
        for (int e = tid; e < G * KC * dk8; e += kThreads) {
            const int c = e % dk8, j = (e / dk8) % KC, g = e / (dk8 * KC);
            uint4 v = make_uint4(0, 0, 0, 0);
            if (j0 + j < kv_hi) v = *reinterpret_cast<const uint4*>(pg + ((size_t)g * a.page + at0 + j) * dk + c * 8);
            *reinterpret_cast<uint4*>(KVs + (size_t)(g * KC + j) * L.dkp + c * 8) = v;
        }
        __syncthreads();
        for (int s = warp; s < G * kc8; s += kThreads / 32) {           // a score tile: the heads of a kv head x 8 keys
            const int g = s / kc8, nt = s % kc8;
            float c4[4] = {0.f, 0.f, 0.f, 0.f};
            const T* qa = Qs + (size_t)(g * kRows + (lane & 15)) * L.dkp + (lane >> 4) * 8;
            const T* kb = KVs + (size_t)(g * KC + nt * 8 + (lane & 7)) * L.dkp + ((lane >> 3) & 1) * 8;
            for (int kk = 0; kk < dk; kk += 16) {
                unsigned af[4], bf[2];
                ldsm_x4(af, qa + kk);
                ldsm_x2(bf, kb + kk);
                mma_16816(c4, af, bf);
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int row = (lane >> 2) + 8 * r;
                if (row < per_kv) {
                    const int h = g * per_kv + row;
                    float w2[2];
#pragma unroll
                    for (int cc = 0; cc < 2; ++cc) {
                        const int j = nt * 8 + 2 * (lane & 3) + cc;
                        float w = 0.f;
                        if (j0 + j < kv_hi) {
                            float sc = c4[2 * r + cc] * a.scale;
                            if (cap) sc = a.softcap * (1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * sc * inv_cap)));
                            w = __fdividef(1.0f, 1.0f + __expf(-(sc + pbs[h])));
                        }
                        w2[cc] = w;
                    }
                    *reinterpret_cast<float2*>(Ss + (size_t)h * L.ssp + nt * 8 + 2 * (lane & 3)) = make_float2(w2[0], w2[1]);
                }
            }
        }
        __syncthreads();
        for (int e = tid; e < G * KC * dv8; e += kThreads) {
            const int c = e % dv8, j = (e / dv8) % KC, g = e / (dv8 * KC);
            uint4 v = make_uint4(0, 0, 0, 0);
            if (j0 + j < kv_hi) v = *reinterpret_cast<const uint4*>(pg + (size_t)G * a.page * dk + ((size_t)g * a.page + at0 + j) * dv + c * 8);
            *reinterpret_cast<uint4*>(KVs + (size_t)(g * KC + j) * L.dvp + c * 8) = v;
        }
        for (int e = tid; e < (L.hpad / 8) * KC; e += kThreads) {         // the mix: eight heads a thread at one key
            const int j = e % KC, hc = e / KC;
            float m[8];
#pragma unroll
            for (int x = 0; x < 8; ++x) m[x] = 0.f;
            const float* tp = Ts + hc * 8;
            for (int g = 0; g < H; ++g) {
                const float sv = Ss[(size_t)g * L.ssp + j];
                const float4 t0 = *reinterpret_cast<const float4*>(tp + (size_t)g * L.hpad);
                const float4 t1 = *reinterpret_cast<const float4*>(tp + (size_t)g * L.hpad + 4);
                m[0] += t0.x * sv; m[1] += t0.y * sv; m[2] += t0.z * sv; m[3] += t0.w * sv;
                m[4] += t1.x * sv; m[5] += t1.y * sv; m[6] += t1.z * sv; m[7] += t1.w * sv;
            }
#pragma unroll
            for (int x = 0; x < 8; ++x) {
                const int h = hc * 8 + x;
                if (h < H) Ms[(size_t)((h / per_kv) * kRows + h % per_kv) * L.msp + j] = __float2bfloat16_rn(m[x]);
            }
        }
        __syncthreads();
#pragma unroll
        for (int x = 0; x < NT; ++x) {
            const int t = warp * NT + x;
            if (t < own_tiles) {
                const int g = t / dv8, nt = t % dv8;
                const T* ma = Ms + (size_t)(g * kRows + (lane & 15)) * L.msp + (lane >> 4) * 8;
                const T* vb = KVs + (size_t)(g * KC + (lane & 15)) * L.dvp + nt * 8;
                for (int kk = 0; kk < KC; kk += 16) {
                    unsigned af[4], bf[2];
                    ldsm_x4(af, ma + kk);
                    ldsm_x2_trans(bf, vb + (size_t)kk * L.dvp);
                    mma_16816(acc[x], af, bf);
                }
            }
        }
    }
#pragma unroll
    for (int x = 0; x < NT; ++x) {
        const int t = warp * NT + x;
        if (t < own_tiles) {
            const int g = t / dv8, nt = t % dv8;
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int row = (lane >> 2) + 8 * r;
                if (row < per_kv) {
                    const size_t at = (size_t)first * HD + (size_t)(g * per_kv + row) * dv + nt * 8 + 2 * (lane & 3);
                    if (a.ranges > 1) {
                        *reinterpret_cast<float2*>(a.partial + (size_t)blockIdx.y * a.n_tokens * HD + at) = make_float2(acc[x][2 * r], acc[x][2 * r + 1]);
                    } else {
                        *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<T*>(a.out) + at) = __floats2bfloat162_rn(acc[x][2 * r], acc[x][2 * r + 1]);
                    }
                }
            }
        }
    }
}

// (KC, NT) of the single-token tensor-core kernel for a shape, or false when it does not take it
static bool rows_plan(int H, int G, int dk, int dv, int page, int* KC_out, int* NT_out, size_t* smem_out) {
    if (dk % 16 || dv % 8 || H % G || H / G > kRows) return false;
    const int nt = (G * (dv / 8) + kThreads / 32 - 1) / (kThreads / 32);
    if (nt > 16) return false;
    const size_t room[3] = {72 * 1024, 110 * 1024, 200 * 1024};      // three blocks an SM if a chunk allows, else two, else one
    for (int pass = 0; pass < 3; ++pass)
        for (int KC = 32; KC >= 16; KC /= 2) {
            if (page % KC) continue;
            const RowsLayout l = rows_layout(H, G, dk, dv, KC);
            if (l.total <= room[pass]) {
                *KC_out = KC;
                *NT_out = nt <= 2 ? 2 : (nt <= 4 ? 4 : (nt <= 8 ? 8 : 16));
                *smem_out = l.total;
                return true;
            }
        }
    return false;
}

// (KC, HG, NT) of the tensor-core kernel for a shape, or false when it does not take it
static bool mma_plan(int H, int G, int dk, int dv, int page, int* KC_out, int* HG_out, int* NT_out, size_t* smem_out) {
    if (dk % 16 || dv % 8 || H % G) return false;
    for (int HG = 1; HG <= H; HG *= 2) {
        if (H % HG) break;
        const int own_tiles = (H / HG) * (dv / 8);
        const int nt = (own_tiles + kThreadsMma / 32 - 1) / (kThreadsMma / 32);
        if (nt > 8) continue;
        for (int KC = 32; KC >= 16; KC /= 2) {
            if (page % KC) continue;
            const MmaLayout l = mma_layout(H, G, dk, dv, KC, HG);
            if (l.total <= 226 * 1024) {      // of the 227 KB a block can have

                *KC_out = KC;
                *HG_out = HG;
                *NT_out = nt <= 2 ? 2 : (nt <= 4 ? 4 : 8);
                *smem_out = l.total;
                return true;
            }
        }
    }
    return false;
}

// out[n, :] = the ranges' partial outputs added in order; rows of no sequence get zeros
template <typename T>
__global__ void add_ranges_kernel(const float* __restrict__ partial, T* __restrict__ out, const int* __restrict__ token_seq,
                                  int n_tokens, int HD, int ranges) {
    const int n = blockIdx.y;
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= HD) return;
    float s = 0.f;
    if (token_seq[n] >= 0)
        for (int r = 0; r < ranges; ++r) s += partial[((size_t)r * n_tokens + n) * HD + e];
    out[(size_t)n * HD + e] = from_f32<T>(s);
}

struct SigmoidAttnPlan {
    int BQ, KC, acc;
    size_t smem;
};

template <typename T>
static size_t smem_bytes(int H, int G, int dk, int dv, int BQ, int KC) {
    const int dkp = padded<T>(dk), dvp = padded<T>(dv), kvp = dkp > dvp ? dkp : dvp;
    return ((size_t)(H * H + 3) / 4 * 4 + (H + 3) / 4 * 4 + 2 * (size_t)H * BQ * KC) * sizeof(float) +
           ((size_t)H * BQ * dkp + (size_t)G * KC * kvp) * sizeof(T);
}

// BQ: as many query rows as the registers hold outputs for (64 a thread at most), 8 at most, no more than the step
// has; KC: 64, 32 or 16 keys, the most that fits the shared memory.
template <typename T>
static bool plan_for(int H, int G, int dk, int dv, int max_q_len, int page, SigmoidAttnPlan* p) {
    const size_t limit = 200 * 1024;
    int BQ = 8;
    while (BQ > 1 && ((size_t)H * BQ * dv > (size_t)64 * kThreads || BQ / 2 >= max_q_len)) BQ /= 2;
    if ((size_t)H * BQ * dv > (size_t)64 * kThreads) return false;
    // single rows (decoding) are bound by the latency of their loads: a chunk small enough for four blocks an SM, if any
    const size_t roomy = max_q_len == 1 ? 56 * 1024 : limit;
    for (int pass = 0; pass < 2; ++pass)
    for (int bq = BQ; bq >= 1; bq /= 2) {
        for (int KC = 64; KC >= 16; KC /= 2) {
            if (KC > page || page % KC) continue;
            const size_t s = smem_bytes<T>(H, G, dk, dv, bq, KC);
            if (s <= (pass == 0 ? roomy : limit)) {
                BQ = bq;
                const size_t outs = ((size_t)H * BQ * dv + kThreads - 1) / kThreads;
                p->BQ = BQ;
                p->KC = KC;
                p->acc = outs <= 4 ? 4 : (outs <= 16 ? 16 : 64);
                p->smem = s;
                return true;
            }
        }
    }
    return false;
}

BLM_API int blm_sigmoid_attention_takes(int dtype, int H, int G, int dk, int dv, int page) {
    SigmoidAttnPlan p;
    if (H < 1 || G < 1 || H % G) return 0;
    return dtype == BLM_F32 ? plan_for<float>(H, G, dk, dv, 1, page, &p) : plan_for<__nv_bfloat16>(H, G, dk, dv, 1, page, &p);
}

static int finish_ranges_bf16(const SigmoidAttnArgs& a, const int* token_seq, cudaStream_t stream);

// bfloat16 steps whose shape the tensor-core kernel takes (single tokens too: a tile then has one row, which costs the
// tensor cores nothing that matters beside the keys' and values' way in); returns -1 when it does not
static int launch_sigmoid_attention_mma(SigmoidAttnArgs a, int max_q_len, const int* token_seq, cudaStream_t stream) {
    int KC, HG, NT;
    size_t smem;
    if ((((size_t)a.q | (size_t)a.pool | (size_t)a.out) & 15) != 0) return -1;
    if (max_q_len == 1) {            // single tokens: the heads of a key/value head are a tile's rows
        if (!rows_plan(a.H, a.G, a.dk, a.dv, a.page, &KC, &NT, &smem)) return -1;
        a.BQ = 1;
        a.KC = KC;
        a.q_tiles = 1;
        BLM_REQUIRE(a.ranges <= 65535, "sigmoid_attention: grid too large");
        dim3 grid(a.n_seqs, a.ranges);
#define BLM_SAR(N)                                                                                                       \
    {                                                                                                                    \
        auto k = sigmoid_attn_rows_kernel<N>;                                                                            \
        if (smem > 48 * 1024) {                                                                                          \
            cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);             \
            if (e != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "sigmoid_attention: %s", cudaGetErrorString(e));       \
        }                                                                                                                \
        k<<<grid, kThreads, smem, stream>>>(a);                                                                          \
    }
        if (NT == 2) BLM_SAR(2) else if (NT == 4) BLM_SAR(4) else if (NT == 8) BLM_SAR(8) else BLM_SAR(16)
#undef BLM_SAR
        int rc = blm_check_launch("sigmoid_attention (single tokens, tensor cores)");
        if (rc != BLM_OK || a.ranges == 1) return rc;
        return finish_ranges_bf16(a, token_seq, stream);
    }
    if (max_q_len < kMmaMinRows || !mma_plan(a.H, a.G, a.dk, a.dv, a.page, &KC, &HG, &NT, &smem)) return -1;
    a.BQ = kRows;
    a.KC = KC;
    a.q_tiles = (max_q_len + kRows - 1) / kRows;
    BLM_REQUIRE((long long)a.n_seqs * a.q_tiles <= 0x7fffffffLL && a.ranges <= 65535 && HG <= 65535, "sigmoid_attention: grid too large");
    dim3 grid(a.n_seqs * a.q_tiles, a.ranges, HG);
#define BLM_SAM(N)                                                                                                       \
    {                                                                                                                    \
        auto k = sigmoid_attn_mma_kernel<N>;                                                                             \
        if (smem > 48 * 1024) {                                                                                          \
            cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);             \
            if (e != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "sigmoid_attention: %s", cudaGetErrorString(e));       \
        }                                                                                                                \
        k<<<grid, kThreadsMma, smem, stream>>>(a, HG);                                                                     \
    }
    if (NT == 2) BLM_SAM(2) else if (NT == 4) BLM_SAM(4) else BLM_SAM(8)
#undef BLM_SAM
    int rc = blm_check_launch("sigmoid_attention (tensor cores)");
    if (rc != BLM_OK || a.ranges == 1) return rc;
    return finish_ranges_bf16(a, token_seq, stream);
}

template <typename T>
static int launch_sigmoid_attention(SigmoidAttnArgs a, int max_q_len, const int* token_seq, cudaStream_t stream) {
    SigmoidAttnPlan p;
    BLM_REQUIRE(plan_for<T>(a.H, a.G, a.dk, a.dv, max_q_len, a.page, &p),
                "sigmoid_attention: %d heads of %d + %d lanes do not fit this kernel's registers and shared memory", a.H, a.dk, a.dv);
    a.BQ = p.BQ;
    a.KC = p.KC;
    a.q_tiles = (max_q_len + p.BQ - 1) / p.BQ;
    BLM_REQUIRE((long long)a.n_seqs * a.q_tiles <= 0x7fffffffLL && a.ranges <= 65535, "sigmoid_attention: grid too large");
    dim3 grid(a.n_seqs * a.q_tiles, a.ranges);
#define BLM_SA(ACC)                                                                                                      \
    {                                                                                                                    \
        auto k = sigmoid_attn_kernel<T, ACC>;                                                                            \
        if (p.smem > 48 * 1024) {                                                                                        \
            cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem);           \
            if (e != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "sigmoid_attention: %s", cudaGetErrorString(e));       \
        }                                                                                                                \
        k<<<grid, kThreads, p.smem, stream>>>(a);                                                                        \
    }
    if (p.acc == 4) BLM_SA(4) else if (p.acc == 16) BLM_SA(16) else BLM_SA(64)
#undef BLM_SA
    int rc = blm_check_launch("sigmoid_attention");
    if (rc != BLM_OK || a.ranges == 1) return rc;
    const int HD = a.H * a.dv;
    dim3 grid2((HD + 255) / 256, a.n_tokens);
    add_ranges_kernel<T><<<grid2, 256, 0, stream>>>(a.partial, (T*)a.out, token_seq, a.n_tokens, HD, a.ranges);
    return blm_check_launch("sigmoid_attention (ranges)");
}

static int finish_ranges_bf16(const SigmoidAttnArgs& a, const int* token_seq, cudaStream_t stream) {
    const int HD = a.H * a.dv;
    dim3 grid2((HD + 255) / 256, a.n_tokens);
    add_ranges_kernel<__nv_bfloat16><<<grid2, 256, 0, stream>>>(a.partial, (__nv_bfloat16*)a.out, token_seq, a.n_tokens, HD, a.ranges);
    return blm_check_launch("sigmoid_attention (ranges)");
}

BLM_API int blm_sigmoid_attention(const void* q, const void* pool, int dtype, const int* block_table, int table_stride,
                                  const int* cu_seqlens, const int* slot_of_seq, const int* start_pos, const int* token_seq,
                                  const float* talk, const float* head_bias, void* out, float* partial, int n_tokens, int n_seqs,
                                  int max_q_len, int H, int G, int dk, int dv, int page, int ranges, float scale, float softcap,
                                  int scalar_only, cudaStream_t stream) {
    if (n_tokens == 0 || n_seqs == 0) return BLM_OK;
    BLM_REQUIRE(H > 0 && G > 0 && H % G == 0 && dk > 0 && dv > 0 && max_q_len > 0, "sigmoid_attention: bad sizes");
    BLM_REQUIRE(ranges >= 1 && (ranges == 1 || partial != nullptr), "sigmoid_attention: several key ranges need a workspace");
    BLM_REQUIRE(n_tokens <= 65535, "sigmoid_attention: a step of %d rows; this kernel takes 65,535", n_tokens);
    SigmoidAttnArgs a;
    a.q = q; a.pool = pool; a.block_table = block_table; a.table_stride = table_stride; a.cu_seqlens = cu_seqlens;
    a.slot_of_seq = slot_of_seq; a.start_pos = start_pos; a.talk = talk; a.head_bias = head_bias; a.out = out; a.partial = partial;
    a.n_tokens = n_tokens; a.n_seqs = n_seqs; a.q_tiles = 0; a.H = H; a.G = G; a.dk = dk; a.dv = dv; a.page = page; a.BQ = 0; a.KC = 0;
    a.ranges = ranges; a.scale = scale; a.softcap = softcap;
    if (dtype == BLM_F32) return launch_sigmoid_attention<float>(a, max_q_len, token_seq, stream);
    if (dtype == BLM_BF16) {
        if (!scalar_only) {
            const int rc = launch_sigmoid_attention_mma(a, max_q_len, token_seq, stream);
            if (rc >= 0) return rc;
        }
        return launch_sigmoid_attention<__nv_bfloat16>(a, max_q_len, token_seq, stream);
    }
    return blm_fail(BLM_BAD_ARGUMENT, "sigmoid_attention: dtype %d", dtype);
}
