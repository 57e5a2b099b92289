// Latent attention: queries and keys/values that go through low-rank latents, one latent row per token in
// the paged cache, shared by all heads.
//
// Per token the mixer keeps a row of R = kv_rank + rot_dim elements: the normed latent c (kv_rank) and one
// rotated key part (rot_dim) that all heads share.  A head's unrotated key is W_uk[h] c and its value
// W_uv[h] c, so the score of query (t, h) against key j is
//
//     s = ((W_uk[h]^T q_nope) . c_j + q_rot . k_rot_j) * scale
//
// and the head's output W_uv[h] (sum_j p_j c_j): with the query carried into the latent space first
// ("absorbed"), attention runs over the cached rows as they are, as one key/value head of width R (keys) and
// kv_rank (values = the first kv_rank elements of the same row) for all query heads, and nothing per head is
// ever expanded per key.  The two per-head products are grouped products of the framework (the heads take
// the place of experts); for them the queries and the attention output are laid out head-major,
// [head][token][...].
//
// Kernels of this file:
//   latent_prep     norms of the two latents, rotation of the shared key part, cache write (one pass over
//                   the down-projection's output)
//   latent_q_split  the up-projected query: unrotated parts to head-major rows, rotated parts turned
//   latent_attn     attention over the latent rows, float32 arithmetic: a sliding window (a query at position p
//                   sees p - window < j <= p; 0 = all), and a sink per head: exp(sink[h]) joins the softmax's
//                   denominator, without a key or a value
//   heads_to_rows   [head][token][d] -> [token][head * d]
//
// Angles: position * frequency and its sine and cosine are formed in float64 from float64 frequencies (the
// host computes them, ramp of a long-context scaling included) and rounded once; `magnitude` multiplies both.
// Pairs are interleaved: (2i, 2i + 1), i < rot_pairs; elements behind 2 * rot_pairs pass unchanged.
#include "common.cuh"

__device__ __forceinline__ float block_sum_256(float v, float* part) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) tot += part[k];
    __syncthreads();
    return tot;
}

// ---------------------------------------------------------------------------
// dqkv [T, q_rank + kv_rank + rot_dim] float32: the stacked down-projections of a token.
//   cq[t]            = rmsnorm(dqkv[t, :q_rank]) * wq                       -> cq_out [T, q_rank]
//   row[:kv_rank]    = rmsnorm(dqkv[t, q_rank : q_rank + kv_rank]) * wkv    -> the token's cache row
//   row[kv_rank:]    = rotate(dqkv[t, q_rank + kv_rank :], position)
template <typename TO, typename TW>
__global__ void __launch_bounds__(256) latent_prep_kernel(
    const float* __restrict__ dqkv, const int* __restrict__ positions, const double* __restrict__ freq,
    float magnitude, const TW* __restrict__ wq, const TW* __restrict__ wkv, float eps, TO* __restrict__ cq_out,
    TO* __restrict__ pool, const int* __restrict__ slots, int q_rank, int kv_rank, int rot_dim, int rot_pairs,
    int write) {
    __shared__ float part[8];
    pdl_entry();
    pdl_trigger();
    const int t = blockIdx.x;
    const int width = q_rank + kv_rank + rot_dim;
    const float* src = dqkv + static_cast<size_t>(t) * width;
    float sq = 0.f, sk = 0.f;
    for (int j = threadIdx.x; j < q_rank; j += 256) sq = fmaf(src[j], src[j], sq);
    for (int j = threadIdx.x; j < kv_rank; j += 256) sk = fmaf(src[q_rank + j], src[q_rank + j], sk);
    sq = block_sum_256(sq, part);
    sk = block_sum_256(sk, part);
    const float scale_q = 1.0f / sqrtf(sq / static_cast<float>(q_rank) + eps);
    const float scale_k = 1.0f / sqrtf(sk / static_cast<float>(kv_rank) + eps);
    TO* cq = cq_out + static_cast<size_t>(t) * q_rank;
    for (int j = threadIdx.x; j < q_rank; j += 256) cq[j] = from_f<TO>(src[j] * scale_q * to_f(wq[j]));
    if (!write) return;
    TO* row = pool + static_cast<size_t>(slots[t]) * (kv_rank + rot_dim);
    for (int j = threadIdx.x; j < kv_rank; j += 256) row[j] = from_f<TO>(src[q_rank + j] * scale_k * to_f(wkv[j]));
    const float* kr = src + q_rank + kv_rank;
    const double pos = static_cast<double>(positions[t]);
    for (int i = threadIdx.x; i < rot_pairs; i += 256) {
        double s, c;
        sincos(pos * freq[i], &s, &c);
        const float cs = static_cast<float>(c) * magnitude, sn = static_cast<float>(s) * magnitude;
        const float u = kr[2 * i], v = kr[2 * i + 1];
        row[kv_rank + 2 * i] = from_f<TO>(u * cs - v * sn);
        row[kv_rank + 2 * i + 1] = from_f<TO>(v * cs + u * sn);
    }
    for (int j = 2 * rot_pairs + threadIdx.x; j < rot_dim; j += 256) row[kv_rank + j] = from_f<TO>(kr[j]);
}

extern "C" int locus_latent_prep(const float* dqkv, const int* positions, const double* freq, float magnitude,
                                 const void* wq, const void* wkv, int w_dt, float eps, void* cq_out, void* pool,
                                 int dt, const int* slots, int T, int q_rank, int kv_rank, int rot_dim,
                                 int rot_pairs, int write, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (q_rank <= 0 || kv_rank <= 0 || rot_dim < 0 || rot_pairs < 0 || 2 * rot_pairs > rot_dim) return LOCUS_ERR_UNSUPPORTED;
    if (rot_pairs > 0 && freq == nullptr) return LOCUS_ERR_UNSUPPORTED;
#define PREP(TO, TW)                                                                                              \
    locus_launch(latent_prep_kernel<TO, TW>, T, 256, 0, stream, dqkv, positions, freq, magnitude,                  \
                 static_cast<const TW*>(wq), static_cast<const TW*>(wkv), eps, static_cast<TO*>(cq_out),           \
                 static_cast<TO*>(pool), slots, q_rank, kv_rank, rot_dim, rot_pairs, write)
    if (dt == LOCUS_DT_BF16 && w_dt == LOCUS_DT_BF16) PREP(bf16, bf16);
    else if (dt == LOCUS_DT_F32 && w_dt == LOCUS_DT_F32) PREP(float, float);
    else if (dt == LOCUS_DT_F32 && w_dt == LOCUS_DT_BF16) PREP(float, bf16);
    else if (dt == LOCUS_DT_BF16 && w_dt == LOCUS_DT_F32) PREP(bf16, float);
    else return LOCUS_ERR_UNSUPPORTED;
#undef PREP
    return locus_launch_status();
}

// ---------------------------------------------------------------------------
// q [T, H * (dn + dr)], head by head [dn unrotated | dr rotated]:
//   q_nope_hm [H, T, dn]   the unrotated parts, head-major (the rows of the grouped product with W_uk^T)
//   q_rot     [T, H, dr]   the rotated parts, turned by the token's position
template <typename TA>
__global__ void __launch_bounds__(256) latent_q_split_kernel(
    const TA* __restrict__ q, const int* __restrict__ positions, const double* __restrict__ freq, float magnitude,
    TA* __restrict__ q_nope_hm, TA* __restrict__ q_rot, int T, int H, int dn, int dr, int rot_pairs) {
    extern __shared__ float cs_tab[];  // [rot_pairs][2]
    pdl_entry();
    pdl_trigger();
    const int t = blockIdx.x;
    const double pos = static_cast<double>(positions[t]);
    for (int i = threadIdx.x; i < rot_pairs; i += 256) {
        double s, c;
        sincos(pos * freq[i], &s, &c);
        cs_tab[2 * i] = static_cast<float>(c) * magnitude;
        cs_tab[2 * i + 1] = static_cast<float>(s) * magnitude;
    }
    __syncthreads();
    const int hw = dn + dr;
    const TA* src = q + static_cast<size_t>(t) * H * hw;
    for (int i = threadIdx.x; i < H * dn; i += 256) {
        const int h = i / dn, d = i % dn;
        q_nope_hm[(static_cast<size_t>(h) * T + t) * dn + d] = src[h * hw + d];
    }
    TA* dst = q_rot + static_cast<size_t>(t) * H * dr;
    const int half = dr / 2;  // pairs of a head, turned or not
    for (int i = threadIdx.x; i < H * half; i += 256) {
        const int h = i / half, p = i % half;
        const float u = to_f(src[h * hw + dn + 2 * p]), v = to_f(src[h * hw + dn + 2 * p + 1]);
        float a = u, b = v;
        if (p < rot_pairs) {
            const float cs = cs_tab[2 * p], sn = cs_tab[2 * p + 1];
            a = u * cs - v * sn;
            b = v * cs + u * sn;
        }
        dst[h * dr + 2 * p] = from_f<TA>(a);
        dst[h * dr + 2 * p + 1] = from_f<TA>(b);
    }
    if (dr & 1)
        for (int h = threadIdx.x; h < H; h += 256) dst[h * dr + dr - 1] = src[h * hw + dn + dr - 1];
}

extern "C" int locus_latent_q_split(const void* q, int dt, const int* positions, const double* freq,
                                    float magnitude, void* q_nope_hm, void* q_rot, int T, int H, int dn, int dr,
                                    int rot_pairs, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || dn <= 0 || dr < 0 || rot_pairs < 0 || 2 * rot_pairs > dr) return LOCUS_ERR_UNSUPPORTED;
    if (rot_pairs > 0 && freq == nullptr) return LOCUS_ERR_UNSUPPORTED;
    const size_t smem = sizeof(float) * 2 * (rot_pairs > 0 ? rot_pairs : 1);
    if (smem > 48 * 1024) return LOCUS_ERR_UNSUPPORTED;
    if (dt == LOCUS_DT_BF16)
        locus_launch(latent_q_split_kernel<bf16>, T, 256, smem, stream, static_cast<const bf16*>(q), positions, freq,
                     magnitude, static_cast<bf16*>(q_nope_hm), static_cast<bf16*>(q_rot), T, H, dn, dr, rot_pairs);
    else if (dt == LOCUS_DT_F32)
        locus_launch(latent_q_split_kernel<float>, T, 256, smem, stream, static_cast<const float*>(q), positions, freq,
                     magnitude, static_cast<float*>(q_nope_hm), static_cast<float*>(q_rot), T, H, dn, dr, rot_pairs);
    else
        return LOCUS_ERR_UNSUPPORTED;
    return locus_launch_status();
}

// ---------------------------------------------------------------------------
// src [H, T, d] -> out [T, H * d]
template <typename TA>
__global__ void __launch_bounds__(256) heads_to_rows_kernel(const TA* __restrict__ src, TA* __restrict__ out, int T,
                                                            int H, int d) {
    pdl_entry();
    pdl_trigger();
    const int t = blockIdx.x;
    TA* dst = out + static_cast<size_t>(t) * H * d;
    for (int i = threadIdx.x; i < H * d; i += 256) {
        const int h = i / d, e = i % d;
        dst[i] = src[(static_cast<size_t>(h) * T + t) * d + e];
    }
}

extern "C" int locus_heads_to_rows(const void* src, int dt, void* out, int T, int H, int d, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || d <= 0) return LOCUS_ERR_UNSUPPORTED;
    if (dt == LOCUS_DT_BF16)
        locus_launch(heads_to_rows_kernel<bf16>, T, 256, 0, stream, static_cast<const bf16*>(src), static_cast<bf16*>(out), T, H, d);
    else if (dt == LOCUS_DT_F32)
        locus_launch(heads_to_rows_kernel<float>, T, 256, 0, stream, static_cast<const float*>(src), static_cast<float*>(out), T, H, d);
    else
        return LOCUS_ERR_UNSUPPORTED;
    return locus_launch_status();
}

// ---------------------------------------------------------------------------
// Attention over the latent rows on the CUDA cores, float32 arithmetic throughout.
struct LatentArgs {
    const void* q_abs;       // [H, T, kv_rank] head-major: the unrotated queries carried into the latent space
    const void* q_rot;       // [T, H, rot_dim]
    const void* pool;        // this layer's pages: [n_pages][page_tokens][kv_rank + rot_dim]
    const float* sink;       // [H] or null
    void* out;               // [H, T, kv_rank] head-major: sum_j p_j c_j
    const int* seg_q0;
    const int* seg_qn;
    const int* seg_ctx;
    const int* block_table;  // [n_seg, table_stride]; entries behind a window may be -1
    int table_stride;
    const int* items;        // [n_items, 2] (segment, first query of a tile of LAT_BQ queries within it)
    int T, H, kv_rank, rot_dim, page_tokens, window;
    float scale;
};

#define LAT_BQ 16
#define LAT_TK 32

template <typename T, int NACC>
__global__ void __launch_bounds__(128) latent_attn_kernel(LatentArgs a) {
    extern __shared__ float smem[];
    const int kvr = a.kv_rank, R = a.kv_rank + a.rot_dim;
    float* qs = smem;                            // [BQ][R]
    float* ks = qs + LAT_BQ * R;                 // [TK][R + 1]
    float* sc = ks + LAT_TK * (R + 1);           // [BQ][TK + 1]
    float* m_s = sc + LAT_BQ * (LAT_TK + 1);     // [BQ]
    float* l_s = m_s + LAT_BQ;                   // [BQ]
    float* al_s = l_s + LAT_BQ;                  // [BQ]
    pdl_entry();
    pdl_trigger();
    // the late tiles of a prompt see the most keys: the grid takes them first, for all heads (its fast index)
    const int item = gridDim.y - 1 - blockIdx.y;
    const int seg = a.items[2 * item], qoff = a.items[2 * item + 1];
    const int h = blockIdx.x;
    const int nq = min(LAT_BQ, a.seg_qn[seg] - qoff);
    const int row0 = a.seg_q0[seg] + qoff;
    const int p0 = a.seg_ctx[seg] + qoff;  // position of the tile's first query
    const int* table = a.block_table + static_cast<size_t>(seg) * a.table_stride;
    const int tid = threadIdx.x;
    const T* qa = static_cast<const T*>(a.q_abs) + (static_cast<size_t>(h) * a.T + row0) * kvr;
    const T* qr = static_cast<const T*>(a.q_rot);
    for (int i = tid; i < LAT_BQ * R; i += 128) {
        const int qi = i / R, d = i % R;
        float v = 0.f;
        if (qi < nq)
            v = d < kvr ? to_f(qa[static_cast<size_t>(qi) * kvr + d])
                        : to_f(qr[(static_cast<size_t>(row0 + qi) * a.H + h) * a.rot_dim + (d - kvr)]);
        qs[i] = v;
    }
    if (tid < LAT_BQ) {
        // the sink is a score of its own in the denominator: the running maximum starts at it, with weight 1
        const bool has = a.sink != nullptr;
        m_s[tid] = has ? a.sink[h] : -INFINITY;
        l_s[tid] = has ? 1.f : 0.f;
    }
    const int t_hi = p0 + nq - 1;
    const int t_lo = a.window > 0 ? max(0, p0 - a.window + 1) : 0;
    const int my_q = tid >> 3, dl = tid & 7;
    float acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
    __syncthreads();

    for (int tile0 = (t_lo / LAT_TK) * LAT_TK; tile0 <= t_hi; tile0 += LAT_TK) {
        for (int i = tid; i < LAT_TK * R; i += 128) {
            const int kj = i / R, d = i % R;
            const int t = tile0 + kj;
            float kv = 0.f;
            if (t >= t_lo && t <= t_hi) {
                const size_t slot = static_cast<size_t>(table[t / a.page_tokens]) * a.page_tokens + t % a.page_tokens;
                kv = to_f(static_cast<const T*>(a.pool)[slot * R + d]);
            }
            ks[kj * (R + 1) + d] = kv;
        }
        __syncthreads();
        for (int i = tid; i < LAT_BQ * LAT_TK; i += 128) {
            const int qi = i / LAT_TK, kj = i % LAT_TK;
            const int t = tile0 + kj, p = p0 + qi;
            float s = -INFINITY;
            if (qi < nq && t <= p && t >= t_lo && (a.window == 0 || t > p - a.window)) {
                float dot = 0.f;
                const float* qrow = qs + qi * R;
                const float* krow = ks + kj * (R + 1);
                for (int d = 0; d < R; ++d) dot = fmaf(qrow[d], krow[d], dot);
                s = dot * a.scale;
            }
            sc[qi * (LAT_TK + 1) + kj] = s;
        }
        __syncthreads();
        if (tid < LAT_BQ) {
            float* row = sc + tid * (LAT_TK + 1);
            float mx = m_s[tid];
            for (int kj = 0; kj < LAT_TK; ++kj) mx = fmaxf(mx, row[kj]);
            float alpha = 1.f, sum = 0.f;
            if (mx == -INFINITY) {
                for (int kj = 0; kj < LAT_TK; ++kj) row[kj] = 0.f;
            } else {
                alpha = expf(m_s[tid] - mx);  // exp(-inf) = 0 on the first live tile
                for (int kj = 0; kj < LAT_TK; ++kj) {
                    const float pexp = expf(row[kj] - mx);
                    row[kj] = pexp;
                    sum += pexp;
                }
            }
            m_s[tid] = mx;
            l_s[tid] = l_s[tid] * alpha + sum;
            al_s[tid] = alpha;
        }
        __syncthreads();
        {
            const float alpha = al_s[my_q];
            const float* prow = sc + my_q * (LAT_TK + 1);
#pragma unroll
            for (int dd = 0; dd < NACC; ++dd) {
                const int d = dl + 8 * dd;
                if (d < kvr) {
                    float v = acc[dd] * alpha;
                    for (int kj = 0; kj < LAT_TK; ++kj) v = fmaf(prow[kj], ks[kj * (R + 1) + d], v);
                    acc[dd] = v;
                }
            }
        }
        __syncthreads();
    }
    if (my_q < nq) {
        const float inv = 1.0f / l_s[my_q];
        T* o = static_cast<T*>(a.out) + (static_cast<size_t>(h) * a.T + row0 + my_q) * kvr;
#pragma unroll
        for (int dd = 0; dd < NACC; ++dd) {
            const int d = dl + 8 * dd;
            if (d < kvr) o[d] = from_f<T>(acc[dd] * inv);
        }
    }
}

template <typename T, int NACC>
static int launch_latent(const LatentArgs& a, int n_items, size_t smem, cudaStream_t stream) {
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(latent_attn_kernel<T, NACC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
        return LOCUS_ERR_UNSUPPORTED;
    locus_launch(latent_attn_kernel<T, NACC>, dim3(a.H, n_items), dim3(128), smem, stream, a);
    return locus_launch_status();
}

// window: 0 = every earlier key.  sink: float32 [H] or null.  kv_rank up to 512, rows of up to 640 elements.
extern "C" int locus_latent_attn(const void* q_abs, const void* q_rot, int dt, const void* pool, const float* sink,
                                 void* out, const int* seg_q0, const int* seg_qn, const int* seg_ctx,
                                 const int* block_table, int table_stride, const int* items, int n_items, int T,
                                 int H, int kv_rank, int rot_dim, int page_tokens, int window, float scale,
                                 cudaStream_t stream) {
    if (n_items <= 0) return 0;
    if (H <= 0 || kv_rank <= 0 || kv_rank > 512 || rot_dim < 0 || page_tokens <= 0 || window < 0 || n_items > 65535)
        return LOCUS_ERR_UNSUPPORTED;
    const int R = kv_rank + rot_dim;
    const size_t smem = sizeof(float) * (static_cast<size_t>(LAT_BQ) * R + LAT_TK * (R + 1) + LAT_BQ * (LAT_TK + 1) + 3 * LAT_BQ);
    if (smem > 200 * 1024) return LOCUS_ERR_UNSUPPORTED;
    LatentArgs a;
    a.q_abs = q_abs; a.q_rot = q_rot; a.pool = pool; a.sink = sink; a.out = out; a.seg_q0 = seg_q0; a.seg_qn = seg_qn;
    a.seg_ctx = seg_ctx; a.block_table = block_table; a.table_stride = table_stride; a.items = items; a.T = T; a.H = H;
    a.kv_rank = kv_rank; a.rot_dim = rot_dim; a.page_tokens = page_tokens; a.window = window; a.scale = scale;
    const int nacc = (kv_rank + 7) / 8;
#define LATENT(TT)                                                                \
    do {                                                                          \
        if (nacc <= 8) return launch_latent<TT, 8>(a, n_items, smem, stream);     \
        if (nacc <= 16) return launch_latent<TT, 16>(a, n_items, smem, stream);   \
        if (nacc <= 32) return launch_latent<TT, 32>(a, n_items, smem, stream);   \
        return launch_latent<TT, 64>(a, n_items, smem, stream);                   \
    } while (0)
    if (dt == LOCUS_DT_BF16) LATENT(bf16);
    if (dt == LOCUS_DT_F32) LATENT(float);
#undef LATENT
    return LOCUS_ERR_UNSUPPORTED;
}
