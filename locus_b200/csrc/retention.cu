// Retention: linear attention with a fixed decay per head, no softmax and no denominator.  Per request and
// head a state S [d, dv] (float32, one per state slot, zero when the request opens) is carried from token to
// token:
//
//     S_t = decay_h * S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t
//
// and a head's o_t is divided by its root mean square, multiplied by silu(g_t) and handed to the output
// projection.  Everything here is float32: the projections arrive as float32 rows
// [q: H*d | k: H*d | v: H*dv | g: H*dv] (k is multiplied by k_scale on the way in).
//
//   retention_scan       a warp owns RET_CW columns of one head's state for one request and walks the request's
//                        new tokens in order.  Lane l keeps the rows l, l + 32, ... of its columns in registers
//                        (up to 8 rows: d <= 256); per token one butterfly sum per column.  The order of every
//                        sum is fixed by d alone, so a token's output does not depend on how the request's
//                        tokens were cut into steps or on what else the step holds.
//   retention_intra /    the same recurrence for long portions, a chunk of 32 tokens at a time as small matrix
//   retention_inter      products (see there)
//   retention_gate_norm  out[t, h, :] = o[t, h, :] / rms(o[t, h, :]) * silu(g[t, h, :])   (a warp per row and head)
#include "common.cuh"

#define RET_CW 4

template <int RPL>
__global__ void __launch_bounds__(128) retention_scan_kernel(
    const float* __restrict__ qkvg, int ld, float* __restrict__ state, const int* __restrict__ state_slots,
    const int* __restrict__ seg_q0, const int* __restrict__ seg_qn, const float* __restrict__ decay, float k_scale,
    float* __restrict__ o_raw, int H, int d, int dv, int col_groups, int qn_below) {
    pdl_entry();
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.x * 4 + (threadIdx.x >> 5);  // (head, column group)
    const int seg = blockIdx.y;
    if (unit >= H * col_groups) return;
    if (qn_below > 0 && seg_qn[seg] >= qn_below) return;  // a long portion: the chunked kernel's
    const int h = unit / col_groups, c0 = (unit % col_groups) * RET_CW;
    const int q0 = seg_q0[seg], qn = seg_qn[seg];
    float* S = state + (static_cast<size_t>(state_slots[seg]) * H + h) * d * dv;
    const float lam = decay[h];
    float s[RPL][RET_CW];
#pragma unroll
    for (int r = 0; r < RPL; ++r) {
        const int i = lane + 32 * r;
#pragma unroll
        for (int c = 0; c < RET_CW; ++c) s[r][c] = (i < d && c0 + c < dv) ? S[static_cast<size_t>(i) * dv + c0 + c] : 0.f;
    }
    const int off_q = h * d, off_k = H * d + h * d, off_v = 2 * H * d + h * dv + c0;
    float qn_[RPL], kn_[RPL], vn_[RET_CW];
    auto fetch = [&](int t) {
        const float* row = qkvg + static_cast<size_t>(q0 + t) * ld;
#pragma unroll
        for (int r = 0; r < RPL; ++r) {
            const int i = lane + 32 * r;
            qn_[r] = i < d ? row[off_q + i] : 0.f;
            kn_[r] = i < d ? row[off_k + i] * k_scale : 0.f;
        }
#pragma unroll
        for (int c = 0; c < RET_CW; ++c) vn_[c] = c0 + c < dv ? row[off_v + c] : 0.f;
    };
    if (qn > 0) fetch(0);
    for (int t = 0; t < qn; ++t) {
        float qq[RPL], kk[RPL], vv[RET_CW];
#pragma unroll
        for (int r = 0; r < RPL; ++r) {
            qq[r] = qn_[r];
            kk[r] = kn_[r];
        }
#pragma unroll
        for (int c = 0; c < RET_CW; ++c) vv[c] = vn_[c];
        if (t + 1 < qn) fetch(t + 1);  // the next token's operands are on their way while this one is worked on
        float part[RET_CW];
#pragma unroll
        for (int c = 0; c < RET_CW; ++c) part[c] = 0.f;
#pragma unroll
        for (int r = 0; r < RPL; ++r) {
#pragma unroll
            for (int c = 0; c < RET_CW; ++c) {
                s[r][c] = fmaf(lam, s[r][c], kk[r] * vv[c]);
                part[c] = fmaf(s[r][c], qq[r], part[c]);
            }
        }
#pragma unroll
        for (int c = 0; c < RET_CW; ++c) part[c] = warp_sum(part[c]);
        if (lane < RET_CW && c0 + lane < dv) {
            float v = part[0];
#pragma unroll
            for (int c = 1; c < RET_CW; ++c)
                if (lane == c) v = part[c];
            o_raw[static_cast<size_t>(q0 + t) * H * dv + h * dv + c0 + lane] = v;
        }
    }
#pragma unroll
    for (int r = 0; r < RPL; ++r) {
        const int i = lane + 32 * r;
#pragma unroll
        for (int c = 0; c < RET_CW; ++c)
            if (i < d && c0 + c < dv) S[static_cast<size_t>(i) * dv + c0 + c] = s[r][c];
    }
}

// qkvg [T, ld] float32 with the columns [q | k | v | g]; state [n_slots, H, d, dv] float32; decay [H] float32;
// o_raw [T, H * dv] float32.  d <= 256.  qn_below > 0: only the segments with fewer new tokens than that (the
// others are locus_retention_chunked's).
extern "C" int locus_retention_scan(const float* qkvg, int ld, float* state, const int* state_slots,
                                    const int* seg_q0, const int* seg_qn, int n_seg, const float* decay,
                                    float k_scale, float* o_raw, int H, int d, int dv, int qn_below,
                                    cudaStream_t stream) {
    if (n_seg <= 0) return 0;
    if (H <= 0 || d <= 0 || d > 256 || dv <= 0 || n_seg > 65535 || ld < 2 * H * d + 2 * H * dv) return LOCUS_ERR_UNSUPPORTED;
    const int col_groups = (dv + RET_CW - 1) / RET_CW;
    const dim3 grid((H * col_groups + 3) / 4, n_seg);
    const int rpl = (d + 31) / 32;
#define SCAN(R)                                                                                                 \
    locus_launch(retention_scan_kernel<R>, grid, dim3(128), 0, stream, qkvg, ld, state, state_slots, seg_q0,    \
                 seg_qn, decay, k_scale, o_raw, H, d, dv, col_groups, qn_below)
    if (rpl <= 1) SCAN(1);
    else if (rpl <= 2) SCAN(2);
    else if (rpl <= 4) SCAN(4);
    else SCAN(8);
#undef SCAN
    return locus_launch_status();
}

// ---------------------------------------------------------------------------
// Long portions, chunk by chunk: with the tokens of a chunk of C = 32 as rows of Q, K (scaled) and V,
//
//     O = (Q K^T * D) V + diag(decay^(i+1)) Q S,        D[i][j] = decay^(i-j) for j <= i, else 0
//     S <- decay^n S + (K * decay^(n-1-j))^T V          (n: the chunk's tokens)
//
// which is the recurrence above summed in another order (float32 FMAs on the CUDA cores; the powers of the decay by
// repeated multiplication).  Two kernels.  The first term needs no state: retention_intra_kernel forms it for every
// (request, chunk, head) at once and writes it to o_raw.  retention_inter_kernel then walks a request's chunks in
// order: a block owns `cols` (8, 16 or 32: as many as it takes to fill the GPU) columns of one head's state, keeps them
// in shared memory across the chunks, adds the second term to o_raw and moves the state on.  Rows of Q, K and A are
// read four elements at a time (16-byte rows, padded by one 16-byte piece so that lanes that read different rows hit
// different banks); d4 = d rounded up to a multiple of 4, the tail zero.
#define RC_CHUNK 32

__global__ void __launch_bounds__(256) retention_intra_kernel(
    const float* __restrict__ qkvg, int ld, const int* __restrict__ seg_q0, const int* __restrict__ seg_qn,
    const float* __restrict__ decay, float k_scale, float* __restrict__ o_raw, int H, int d, int dv, int qn_from) {
    extern __shared__ __align__(16) float rc_smem[];
    __shared__ float pw[RC_CHUNK + 1];
    pdl_entry();
    pdl_trigger();
    const int seg = blockIdx.z, h = blockIdx.y;
    const int qn = seg_qn[seg], t0 = blockIdx.x * RC_CHUNK;
    if (qn < qn_from || t0 >= qn) return;
    const int n = min(RC_CHUNK, qn - t0), q0 = seg_q0[seg];
    const int d4 = (d + 3) & ~3, ldq = d4 + 4, lda = RC_CHUNK + 4, dvp = (dv + 31) & ~31;
    float* Qs = rc_smem;                      // [C][ldq]
    float* Ks = Qs + RC_CHUNK * ldq;          // [C][ldq]
    float* As = Ks + RC_CHUNK * ldq;          // [C][lda]
    float* Vs = As + RC_CHUNK * lda;          // [C][dvp]
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    if (tid == 0) {
        float p = 1.f;
        const float lam = decay[h];
        for (int i = 0; i <= RC_CHUNK; ++i) {
            pw[i] = p;
            p *= lam;
        }
    }
    const int off_q = h * d, off_k = H * d + h * d, off_v = 2 * H * d + h * dv;
    for (int i = tid; i < RC_CHUNK * d4; i += 256) {
        const int j = i / d4, r = i % d4;
        const float* row = qkvg + static_cast<size_t>(q0 + t0 + j) * ld;
        const bool ok = j < n && r < d;
        Qs[j * ldq + r] = ok ? row[off_q + r] : 0.f;
        Ks[j * ldq + r] = ok ? row[off_k + r] * k_scale : 0.f;
    }
    for (int i = tid; i < RC_CHUNK * dvp; i += 256) {
        const int j = i / dvp, c = i % dvp;
        Vs[i] = (j < n && c < dv) ? qkvg[static_cast<size_t>(q0 + t0 + j) * ld + off_v + c] : 0.f;
    }
    __syncthreads();
    {   // A = (Q K^T) * D: rows i = wid + 8 u, column j = lane
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        const float4* kr = reinterpret_cast<const float4*>(Ks + lane * ldq);
        for (int r4 = 0; r4 < d4 / 4; ++r4) {
            const float4 k = kr[r4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float4 q = reinterpret_cast<const float4*>(Qs + (wid + 8 * u) * ldq)[r4];
                acc[u] = fmaf(q.x, k.x, acc[u]);
                acc[u] = fmaf(q.y, k.y, acc[u]);
                acc[u] = fmaf(q.z, k.z, acc[u]);
                acc[u] = fmaf(q.w, k.w, acc[u]);
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = wid + 8 * u;
            As[i * lda + lane] = lane <= i ? acc[u] * pw[i - lane] : 0.f;
        }
    }
    __syncthreads();
    // A V: rows i = wid + 8 u, columns lane + 32 cc
    for (int cc = 0; cc < dvp / 32; ++cc) {
        const int c = lane + 32 * cc;
        float intra[4] = {0.f, 0.f, 0.f, 0.f};
        for (int j4 = 0; j4 < RC_CHUNK / 4; ++j4) {
            const float v0 = Vs[(4 * j4) * dvp + c], v1 = Vs[(4 * j4 + 1) * dvp + c];
            const float v2 = Vs[(4 * j4 + 2) * dvp + c], v3 = Vs[(4 * j4 + 3) * dvp + c];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float4 p = reinterpret_cast<const float4*>(As + (wid + 8 * u) * lda)[j4];
                intra[u] = fmaf(p.x, v0, intra[u]);
                intra[u] = fmaf(p.y, v1, intra[u]);
                intra[u] = fmaf(p.z, v2, intra[u]);
                intra[u] = fmaf(p.w, v3, intra[u]);
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = wid + 8 * u;
            if (i < n && c < dv) o_raw[static_cast<size_t>(q0 + t0 + i) * H * dv + h * dv + c] = intra[u];
        }
    }
}

__global__ void __launch_bounds__(256) retention_inter_kernel(
    const float* __restrict__ qkvg, int ld, float* __restrict__ state, const int* __restrict__ state_slots,
    const int* __restrict__ seg_q0, const int* __restrict__ seg_qn, const float* __restrict__ decay, float k_scale,
    float* __restrict__ o_raw, int H, int d, int dv, int col_groups, int cols, int qn_from) {
    extern __shared__ __align__(16) float rc_smem[];
    pdl_entry();
    pdl_trigger();
    const int seg = blockIdx.y;
    const int qn = seg_qn[seg];
    if (qn < qn_from) return;  // a short portion or a single token: the scan kernel's
    const int h = blockIdx.x / col_groups, c0 = (blockIdx.x % col_groups) * cols;
    const int q0 = seg_q0[seg];
    const int d4 = (d + 3) & ~3, ldq = d4 + 4;
    float* Qs = rc_smem;                      // [C][ldq]
    float* Ks = Qs + RC_CHUNK * ldq;          // [C][ldq]
    float* Vs = Ks + RC_CHUNK * ldq;          // [C][cols]
    float* Ss = Vs + RC_CHUNK * cols;         // [d4][cols]
    float* pw = Ss + d4 * cols;               // [C + 1] powers of the decay
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    // a warp's lanes: `cols` columns times 32 / cols shares of the rows
    const int c = lane % cols, sub = lane / cols, nsub = 32 / cols;
    const float lam = decay[h];
    float* S = state + (static_cast<size_t>(state_slots[seg]) * H + h) * d * dv;
    for (int i = tid; i < d4 * cols; i += 256) {
        const int r = i / cols, cc = i % cols;
        Ss[i] = (r < d && c0 + cc < dv) ? S[static_cast<size_t>(r) * dv + c0 + cc] : 0.f;
    }
    if (tid == 0) {
        float p = 1.f;
        for (int n = 0; n <= RC_CHUNK; ++n) {
            pw[n] = p;
            p *= lam;
        }
    }
    const int off_q = h * d, off_k = H * d + h * d, off_v = 2 * H * d + h * dv + c0;
    const int owners = 8 * nsub;                                   // (warp, share) pairs that split the state's rows
    const int rows_o = ((d4 / 4 + owners - 1) / owners) * 4;       // rows of one of them (a multiple of 4)
    const int r_lo = (wid * nsub + sub) * rows_o, r_hi = min(d4, r_lo + rows_o);
    for (int t0 = 0; t0 < qn; t0 += RC_CHUNK) {
        const int n = min(RC_CHUNK, qn - t0);
        __syncthreads();  // the state and the last chunk's operands are free
        for (int i = tid; i < RC_CHUNK * d4; i += 256) {
            const int j = i / d4, r = i % d4;
            const float* row = qkvg + static_cast<size_t>(q0 + t0 + j) * ld;
            const bool ok = j < n && r < d;
            Qs[j * ldq + r] = ok ? row[off_q + r] : 0.f;
            Ks[j * ldq + r] = ok ? row[off_k + r] * k_scale : 0.f;
        }
        for (int i = tid; i < RC_CHUNK * cols; i += 256) {
            const int j = i / cols, cc = i % cols;
            Vs[i] = (j < n && c0 + cc < dv) ? qkvg[static_cast<size_t>(q0 + t0 + j) * ld + off_v + cc] : 0.f;
        }
        __syncthreads();
        {   // o += decay^(i+1) Q S: rows i = wid + 8 u, column c; the lanes' shares of the rows of S are summed by shuffles
            float inter[4] = {0.f, 0.f, 0.f, 0.f};
            for (int r4 = sub; r4 < d4 / 4; r4 += nsub) {
                const float s0 = Ss[(4 * r4) * cols + c], s1 = Ss[(4 * r4 + 1) * cols + c];
                const float s2 = Ss[(4 * r4 + 2) * cols + c], s3 = Ss[(4 * r4 + 3) * cols + c];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float4 q = reinterpret_cast<const float4*>(Qs + (wid + 8 * u) * ldq)[r4];
                    inter[u] = fmaf(q.x, s0, inter[u]);
                    inter[u] = fmaf(q.y, s1, inter[u]);
                    inter[u] = fmaf(q.z, s2, inter[u]);
                    inter[u] = fmaf(q.w, s3, inter[u]);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                for (int o = cols; o < 32; o <<= 1) inter[u] += __shfl_xor_sync(0xffffffffu, inter[u], o);
                const int i = wid + 8 * u;
                if (sub == 0 && i < n && c0 + c < dv) {
                    float* dst = o_raw + static_cast<size_t>(q0 + t0 + i) * H * dv + h * dv + c0 + c;
                    *dst = fmaf(pw[i + 1], inter[u], *dst);
                }
            }
        }
        __syncthreads();
        // S <- decay^n S + (K * decay^(n-1-j))^T V: this lane's rows, column c
        for (int r0 = r_lo; r0 < r_hi; r0 += 4) {
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            for (int j = 0; j < n; ++j) {
                const float v = Vs[j * cols + c] * pw[n - 1 - j];
                const float4 k = *reinterpret_cast<const float4*>(Ks + j * ldq + r0);
                acc[0] = fmaf(k.x, v, acc[0]);
                acc[1] = fmaf(k.y, v, acc[1]);
                acc[2] = fmaf(k.z, v, acc[2]);
                acc[3] = fmaf(k.w, v, acc[3]);
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) Ss[(r0 + e) * cols + c] = fmaf(pw[n], Ss[(r0 + e) * cols + c], acc[e]);
        }
    }
    __syncthreads();
    for (int i = tid; i < d4 * cols; i += 256) {
        const int r = i / cols, cc = i % cols;
        if (r < d && c0 + cc < dv) S[static_cast<size_t>(r) * dv + c0 + cc] = Ss[i];
    }
}

// The segments with at least qn_from new tokens (arguments as locus_retention_scan); longest_new: the most new tokens
// of a segment of the step (an upper bound will do: it sizes the first kernel's grid).
extern "C" int locus_retention_chunked(const float* qkvg, int ld, float* state, const int* state_slots,
                                       const int* seg_q0, const int* seg_qn, int n_seg, const float* decay,
                                       float k_scale, float* o_raw, int H, int d, int dv, int qn_from, int longest_new,
                                       cudaStream_t stream) {
    if (n_seg <= 0 || longest_new <= 0) return 0;
    if (H <= 0 || d <= 0 || d > 256 || dv <= 0 || n_seg > 65535 || H > 65535 || ld < 2 * H * d + 2 * H * dv || qn_from < 1)
        return LOCUS_ERR_UNSUPPORTED;
    const int d4 = (d + 3) & ~3, dvp = (dv + 31) & ~31;
    const size_t smem1 = sizeof(float) * (2 * RC_CHUNK * (d4 + 4) + RC_CHUNK * (RC_CHUNK + 4) + static_cast<size_t>(RC_CHUNK) * dvp);
    if (smem1 > 200 * 1024) return LOCUS_ERR_UNSUPPORTED;
    if (smem1 > 48 * 1024 &&
        cudaFuncSetAttribute(retention_intra_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem1)) != cudaSuccess)
        return LOCUS_ERR_UNSUPPORTED;
    locus_launch(retention_intra_kernel, dim3((longest_new + RC_CHUNK - 1) / RC_CHUNK, H, n_seg), dim3(256), smem1, stream,
                 qkvg, ld, seg_q0, seg_qn, decay, k_scale, o_raw, H, d, dv, qn_from);
    // as few columns per block as it takes to give every SM a block
    int cols = 32;
    while (cols > 8 && static_cast<long long>(H) * ((dv + cols - 1) / cols) * n_seg < 148) cols >>= 1;
    const int col_groups = (dv + cols - 1) / cols;
    const size_t smem2 = sizeof(float) * (2 * RC_CHUNK * (d4 + 4) + RC_CHUNK * cols + static_cast<size_t>(d4) * cols + RC_CHUNK + 4);
    if (smem2 > 48 * 1024 &&
        cudaFuncSetAttribute(retention_inter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem2)) != cudaSuccess)
        return LOCUS_ERR_UNSUPPORTED;
    locus_launch(retention_inter_kernel, dim3(H * col_groups, n_seg), dim3(256), smem2, stream, qkvg, ld, state,
                 state_slots, seg_q0, seg_qn, decay, k_scale, o_raw, H, d, dv, col_groups, cols, qn_from);
    return locus_launch_status();
}

// ---------------------------------------------------------------------------
template <typename TO>
__global__ void __launch_bounds__(256) retention_gate_norm_kernel(const float* __restrict__ o_raw,
                                                                  const float* __restrict__ qkvg, int ld, int g_off,
                                                                  float eps, TO* __restrict__ out, int n_units, int H,
                                                                  int dv) {
    pdl_entry();
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.x * 8 + (threadIdx.x >> 5);  // (token, head)
    if (unit >= n_units) return;
    const int t = unit / H, h = unit % H;
    const float* o = o_raw + static_cast<size_t>(t) * H * dv + h * dv;
    const float* g = qkvg + static_cast<size_t>(t) * ld + g_off + h * dv;
    float ss = 0.f;
    for (int j = lane; j < dv; j += 32) ss = fmaf(o[j], o[j], ss);
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / static_cast<float>(dv) + eps);
    TO* dst = out + static_cast<size_t>(t) * H * dv + h * dv;
    for (int j = lane; j < dv; j += 32) {
        const float z = g[j];
        dst[j] = from_f<TO>(o[j] * scale * (z / (1.0f + expf(-z))));
    }
}

extern "C" int locus_retention_gate_norm(const float* o_raw, const float* qkvg, int ld, int g_off, float eps,
                                         void* out, int out_dt, int T, int H, int dv, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || dv <= 0) return LOCUS_ERR_UNSUPPORTED;
    const long long units = static_cast<long long>(T) * H;
    if (units > 0x7fffffffLL) return LOCUS_ERR_UNSUPPORTED;
    const int blocks = static_cast<int>((units + 7) / 8);
    if (out_dt == LOCUS_DT_BF16)
        locus_launch(retention_gate_norm_kernel<bf16>, blocks, 256, 0, stream, o_raw, qkvg, ld, g_off, eps,
                     static_cast<bf16*>(out), static_cast<int>(units), H, dv);
    else if (out_dt == LOCUS_DT_F32)
        locus_launch(retention_gate_norm_kernel<float>, blocks, 256, 0, stream, o_raw, qkvg, ld, g_off, eps,
                     static_cast<float*>(out), static_cast<int>(units), H, dv);
    else
        return LOCUS_ERR_UNSUPPORTED;
    return locus_launch_status();
}
