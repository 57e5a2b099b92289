// A gated linear recurrence with a matrix state, shared by the mixers that are one: per request and head a
// state S [d, dvx] (float32, in the request's state slot, zero when the request opens) is carried from token to
// token,
//
//     S_t = keep_t * S_(t-1) + take_t * k_t v_t^T,      o_t = S_t^T (q_t * q_scale),
//
// with keep_t and take_t one float32 number per token and head, made by the caller (a decay and a step size, or
// the stabilised gates of a matrix memory).  q and k of head h are those of its group h / heads_per_group (a
// group of heads may share them); v is the head's own.  With `ones` the state has one column more than v
// (dvx = dv + 1) whose v is 1: that column is the recurrence of k alone (a normaliser), and its o is q . n.
// Everything is float32; q, k and v are columns of float32 row matrices given by pointer, row stride and offset.
//
//   gated_scan      a warp owns REC_CW columns of one head's state for one request and walks the request's new
//                   tokens in order; lane l keeps the rows l, l + 32, ... of its columns in registers (d <= 256).
//                   The order of every sum is fixed by d alone.
//   gated_intra /   the same for long portions, a chunk of 32 tokens at a time as small matrix products:
//   gated_inter     O = (Q K^T * D) V + diag(c) Q S,  D[i][j] = take_j * prod_(j < l <= i) keep_l for j <= i,
//                   c_i = prod_(l <= i) keep_l;  S <- c_(n-1) S + (K * D[n-1][.])^T V.  The products of the keeps
//                   are formed by multiplication (no logarithm, no division: a keep of 0 or 1 is no special case).
//                   The first term needs no state and is formed for every (request, chunk, head) at once; the walk
//                   over a request's chunks keeps `cols` columns of the state in shared memory.
#include "common.cuh"

#define REC_CW 4
#define REC_CHUNK 32

struct RecArgs {
    const float* q;
    const float* k;
    const float* v;
    const float* keep;   // [T, H]
    const float* take;   // [T, H]
    float* state;
    const int* state_slots;
    const int* seg_q0;
    const int* seg_qn;
    float* out;          // [T, ldo]: head h's columns start at h * dvx
    long long slot_stride;
    float q_scale;
    int ldq, off_q, ldk, off_k, ldv, off_v, ldo;
    int H, heads_per_group, d, dv, dvx;
};

template <int RPL>
__global__ void __launch_bounds__(128) gated_scan_kernel(const RecArgs a, int col_groups, int qn_below) {
    pdl_entry();
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.x * 4 + (threadIdx.x >> 5);  // (head, column group)
    const int seg = blockIdx.y;
    if (unit >= a.H * col_groups) return;
    const int qn = a.seg_qn[seg];
    if (qn_below > 0 && qn >= qn_below) return;  // a long portion: the chunked kernels'
    const int h = unit / col_groups, c0 = (unit % col_groups) * REC_CW;
    const int d = a.d, dv = a.dv, dvx = a.dvx, q0 = a.seg_q0[seg];
    float* S = a.state + static_cast<size_t>(a.state_slots[seg]) * a.slot_stride + static_cast<size_t>(h) * d * dvx;
    float s[RPL][REC_CW];
#pragma unroll
    for (int r = 0; r < RPL; ++r) {
        const int i = lane + 32 * r;
#pragma unroll
        for (int c = 0; c < REC_CW; ++c) s[r][c] = (i < d && c0 + c < dvx) ? S[static_cast<size_t>(i) * dvx + c0 + c] : 0.f;
    }
    const int g = h / a.heads_per_group;
    const int off_q = a.off_q + g * d, off_k = a.off_k + g * d, off_v = a.off_v + h * dv;
    float qn_[RPL], kn_[RPL], vn_[REC_CW], keep_n = 0.f, take_n = 0.f;
    auto fetch = [&](int t) {
        const size_t row = static_cast<size_t>(q0 + t);
#pragma unroll
        for (int r = 0; r < RPL; ++r) {
            const int i = lane + 32 * r;
            qn_[r] = i < d ? a.q[row * a.ldq + off_q + i] * a.q_scale : 0.f;
            kn_[r] = i < d ? a.k[row * a.ldk + off_k + i] : 0.f;
        }
#pragma unroll
        for (int c = 0; c < REC_CW; ++c)
            vn_[c] = c0 + c < dv ? a.v[row * a.ldv + off_v + c0 + c] : (c0 + c < dvx ? 1.0f : 0.f);
        keep_n = a.keep[row * a.H + h];
        take_n = a.take[row * a.H + h];
    };
    if (qn > 0) fetch(0);
    for (int t = 0; t < qn; ++t) {
        float qq[RPL], kk[RPL], vv[REC_CW];
        const float keep = keep_n, take = take_n;
#pragma unroll
        for (int r = 0; r < RPL; ++r) {
            qq[r] = qn_[r];
            kk[r] = kn_[r] * take;
        }
#pragma unroll
        for (int c = 0; c < REC_CW; ++c) vv[c] = vn_[c];
        if (t + 1 < qn) fetch(t + 1);  // the next token's operands are on their way while this one is worked on
        float part[REC_CW];
#pragma unroll
        for (int c = 0; c < REC_CW; ++c) part[c] = 0.f;
#pragma unroll
        for (int r = 0; r < RPL; ++r) {
#pragma unroll
            for (int c = 0; c < REC_CW; ++c) {
                s[r][c] = fmaf(keep, s[r][c], kk[r] * vv[c]);
                part[c] = fmaf(s[r][c], qq[r], part[c]);
            }
        }
#pragma unroll
        for (int c = 0; c < REC_CW; ++c) part[c] = warp_sum(part[c]);
        if (lane < REC_CW && c0 + lane < dvx) {
            float o = part[0];
#pragma unroll
            for (int c = 1; c < REC_CW; ++c)
                if (lane == c) o = part[c];
            a.out[static_cast<size_t>(q0 + t) * a.ldo + h * dvx + c0 + lane] = o;
        }
    }
#pragma unroll
    for (int r = 0; r < RPL; ++r) {
        const int i = lane + 32 * r;
#pragma unroll
        for (int c = 0; c < REC_CW; ++c)
            if (i < d && c0 + c < dvx) S[static_cast<size_t>(i) * dvx + c0 + c] = s[r][c];
    }
}

// ---------------------------------------------------------------------------
// The chunk's own term for every (request, chunk, head): o = (Q K^T * D) V.
__global__ void __launch_bounds__(256) gated_intra_kernel(const RecArgs a, int qn_from) {
    extern __shared__ __align__(16) float rc_smem[];
    __shared__ float kp[REC_CHUNK], tk[REC_CHUNK];
    pdl_entry();
    pdl_trigger();
    const int seg = blockIdx.z, h = blockIdx.y;
    const int qn = a.seg_qn[seg], t0 = blockIdx.x * REC_CHUNK;
    if (qn < qn_from || t0 >= qn) return;
    const int n = min(REC_CHUNK, qn - t0), q0 = a.seg_q0[seg];
    const int d = a.d, dv = a.dv, dvx = a.dvx;
    const int d4 = (d + 3) & ~3, ldq = d4 + 4, lda = REC_CHUNK + 4, dvp = (dvx + 31) & ~31;
    float* Qs = rc_smem;                       // [C][ldq]
    float* Ks = Qs + REC_CHUNK * ldq;          // [C][ldq]
    float* As = Ks + REC_CHUNK * ldq;          // [C][lda]
    float* Vs = As + REC_CHUNK * lda;          // [C][dvp]
    float* Dm = Vs + REC_CHUNK * dvp;          // [C][C + 1]
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    if (tid < REC_CHUNK) {
        const bool ok = tid < n;
        kp[tid] = ok ? a.keep[static_cast<size_t>(q0 + t0 + tid) * a.H + h] : 1.f;
        tk[tid] = ok ? a.take[static_cast<size_t>(q0 + t0 + tid) * a.H + h] : 0.f;
    }
    const int g = h / a.heads_per_group;
    const int off_q = a.off_q + g * d, off_k = a.off_k + g * d, off_v = a.off_v + h * dv;
    for (int i = tid; i < REC_CHUNK * d4; i += 256) {
        const int j = i / d4, r = i % d4;
        const size_t row = static_cast<size_t>(q0 + t0 + j);
        const bool ok = j < n && r < d;
        Qs[j * ldq + r] = ok ? a.q[row * a.ldq + off_q + r] * a.q_scale : 0.f;
        Ks[j * ldq + r] = ok ? a.k[row * a.ldk + off_k + r] : 0.f;
    }
    for (int i = tid; i < REC_CHUNK * dvp; i += 256) {
        const int j = i / dvp, c = i % dvp;
        float v = 0.f;
        if (j < n) v = c < dv ? a.v[static_cast<size_t>(q0 + t0 + j) * a.ldv + off_v + c] : (c < dvx ? 1.0f : 0.f);
        Vs[i] = v;
    }
    __syncthreads();
    if (tid < REC_CHUNK) {
        // row i of D, from the diagonal backwards: D[i][j] = take_j * keep_(j+1) * ... * keep_i
        float run = 1.f;
        for (int j = tid; j >= 0; --j) {
            Dm[tid * (REC_CHUNK + 1) + j] = run * tk[j];
            run *= kp[j];
        }
    }
    {   // A = Q K^T: rows i = wid + 8 u, column j = lane
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
        __syncthreads();  // D is complete
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = wid + 8 * u;
            As[i * lda + lane] = lane <= i ? acc[u] * Dm[i * (REC_CHUNK + 1) + lane] : 0.f;
        }
    }
    __syncthreads();
    for (int cc = 0; cc < dvp / 32; ++cc) {
        const int c = lane + 32 * cc;
        float intra[4] = {0.f, 0.f, 0.f, 0.f};
        for (int j4 = 0; j4 < REC_CHUNK / 4; ++j4) {
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
            if (i < n && c < dvx) a.out[static_cast<size_t>(q0 + t0 + i) * a.ldo + h * dvx + c] = intra[u];
        }
    }
}

// The walk over a request's chunks: a block owns `cols` columns of one head's state.
__global__ void __launch_bounds__(256) gated_inter_kernel(const RecArgs a, int col_groups, int cols, int qn_from) {
    extern __shared__ __align__(16) float rc_smem[];
    pdl_entry();
    pdl_trigger();
    const int seg = blockIdx.y;
    const int qn = a.seg_qn[seg];
    if (qn < qn_from) return;  // a short portion or a single token: the scan kernel's
    const int h = blockIdx.x / col_groups, c0 = (blockIdx.x % col_groups) * cols;
    const int q0 = a.seg_q0[seg];
    const int d = a.d, dv = a.dv, dvx = a.dvx;
    const int d4 = (d + 3) & ~3, ldq = d4 + 4;
    float* Qs = rc_smem;                       // [C][ldq]
    float* Ks = Qs + REC_CHUNK * ldq;          // [C][ldq]
    float* Vs = Ks + REC_CHUNK * ldq;          // [C][cols]
    // rows of the state lie lds floats apart: lanes of a warp that read the same column of rows 4 apart (the shares of
    // the rows in Q S) or rows_o apart (the update) then hit different banks (cols 8: 10, cols 16: 20)
    const int lds = cols == 32 ? 32 : cols + cols / 4;
    float* Ss = Vs + REC_CHUNK * cols;         // [d4][lds]
    float* kp = Ss + d4 * lds;                 // [C] the chunk's keeps (1 behind its end)
    float* tk = kp + REC_CHUNK;                // [C] and takes (0 behind its end)
    float* wj = tk + REC_CHUNK;                // [8 warps][C] take_j times the keeps behind j, every warp's own copy
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int c = lane % cols, sub = lane / cols, nsub = 32 / cols;
    float* S = a.state + static_cast<size_t>(a.state_slots[seg]) * a.slot_stride + static_cast<size_t>(h) * d * dvx;
    for (int i = tid; i < d4 * cols; i += 256) {
        const int r = i / cols, cc = i % cols;
        Ss[r * lds + cc] = (r < d && c0 + cc < dvx) ? S[static_cast<size_t>(r) * dvx + c0 + cc] : 0.f;
    }
    const int g = h / a.heads_per_group;
    const int off_q = a.off_q + g * d, off_k = a.off_k + g * d, off_v = a.off_v + h * dv;
    const int owners = 8 * nsub;
    const int rows_o = ((d4 / 4 + owners - 1) / owners) * 4;
    const int r_lo = (wid * nsub + sub) * rows_o, r_hi = min(d4, r_lo + rows_o);
    for (int t0 = 0; t0 < qn; t0 += REC_CHUNK) {
        const int n = min(REC_CHUNK, qn - t0);
        __syncthreads();  // the state and the last chunk's operands are free
        for (int i = tid; i < REC_CHUNK * d4; i += 256) {
            const int j = i / d4, r = i % d4;
            const size_t row = static_cast<size_t>(q0 + t0 + j);
            const bool ok = j < n && r < d;
            Qs[j * ldq + r] = ok ? a.q[row * a.ldq + off_q + r] * a.q_scale : 0.f;
            Ks[j * ldq + r] = ok ? a.k[row * a.ldk + off_k + r] : 0.f;
        }
        for (int i = tid; i < REC_CHUNK * cols; i += 256) {
            const int j = i / cols, cc = i % cols;
            float v = 0.f;
            if (j < n) v = c0 + cc < dv ? a.v[static_cast<size_t>(q0 + t0 + j) * a.ldv + off_v + c0 + cc] : (c0 + cc < dvx ? 1.0f : 0.f);
            Vs[i] = v;
        }
        if (tid < REC_CHUNK) {
            kp[tid] = tid < n ? a.keep[static_cast<size_t>(q0 + t0 + tid) * a.H + h] : 1.f;
            tk[tid] = tid < n ? a.take[static_cast<size_t>(q0 + t0 + tid) * a.H + h] : 0.f;
        }
        __syncthreads();
        // Every warp forms the products of the keeps for itself, lane j those of token j: cum = keep_0 .. keep_j, and
        // w = take_j times the keeps behind j (two scans by shuffles; no warp waits for another).
        float cum = kp[lane], suf = kp[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, cum, o), dn = __shfl_down_sync(0xffffffffu, suf, o);
            if (lane >= o) cum *= up;
            if (lane + o < 32) suf *= dn;
        }
        const float behind = __shfl_down_sync(0xffffffffu, suf, 1);
        float* wj_w = wj + wid * REC_CHUNK;
        wj_w[lane] = tk[lane] * (lane < 31 ? behind : 1.f);   // read below by lanes whose loops differ in length: no shuffles there
        const float cum_last = __shfl_sync(0xffffffffu, cum, n - 1);
        __syncwarp();
        {   // o += c_i Q S: rows i = wid + 8 u, column c; the lanes' shares of the rows of S are summed by shuffles
            float inter[4] = {0.f, 0.f, 0.f, 0.f};
            for (int r4 = sub; r4 < d4 / 4; r4 += nsub) {
                const float s0 = Ss[(4 * r4) * lds + c], s1 = Ss[(4 * r4 + 1) * lds + c];
                const float s2 = Ss[(4 * r4 + 2) * lds + c], s3 = Ss[(4 * r4 + 3) * lds + c];
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
                const float ci = __shfl_sync(0xffffffffu, cum, i);
                if (sub == 0 && i < n && c0 + c < dvx) {
                    float* dst = a.out + static_cast<size_t>(q0 + t0 + i) * a.ldo + h * dvx + c0 + c;
                    *dst = fmaf(ci, inter[u], *dst);
                }
            }
        }
        __syncthreads();
        // S <- c_(n-1) S + (K * w)^T V: this lane's rows, column c
        for (int r0 = r_lo; r0 < r_hi; r0 += 4) {
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            for (int j = 0; j < n; ++j) {
                const float v = Vs[j * cols + c] * wj_w[j];
                const float4 k = *reinterpret_cast<const float4*>(Ks + j * ldq + r0);
                acc[0] = fmaf(k.x, v, acc[0]);
                acc[1] = fmaf(k.y, v, acc[1]);
                acc[2] = fmaf(k.z, v, acc[2]);
                acc[3] = fmaf(k.w, v, acc[3]);
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) Ss[(r0 + e) * lds + c] = fmaf(cum_last, Ss[(r0 + e) * lds + c], acc[e]);
        }
    }
    __syncthreads();
    for (int i = tid; i < d4 * cols; i += 256) {
        const int r = i / cols, cc = i % cols;
        if (r < d && c0 + cc < dvx) S[static_cast<size_t>(r) * dvx + c0 + cc] = Ss[r * lds + cc];
    }
}

static bool rec_args_ok(const RecArgs& a, int n_seg) {
    return a.H > 0 && a.heads_per_group > 0 && a.H % a.heads_per_group == 0 && a.d > 0 && a.d <= 256 && a.dv > 0 &&
           (a.dvx == a.dv || a.dvx == a.dv + 1) && n_seg <= 65535 && a.H <= 65535 && a.ldo >= a.H * a.dvx;
}

static RecArgs rec_args(const float* q, int ldq, int off_q, const float* k, int ldk, int off_k, const float* v, int ldv,
                        int off_v, const float* keep, const float* take, float* state, long long slot_stride,
                        const int* state_slots, const int* seg_q0, const int* seg_qn, float q_scale, float* out, int ldo,
                        int H, int heads_per_group, int d, int dv, int ones) {
    RecArgs a;
    a.q = q; a.k = k; a.v = v; a.keep = keep; a.take = take; a.state = state; a.state_slots = state_slots;
    a.seg_q0 = seg_q0; a.seg_qn = seg_qn; a.out = out; a.slot_stride = slot_stride; a.q_scale = q_scale;
    a.ldq = ldq; a.off_q = off_q; a.ldk = ldk; a.off_k = off_k; a.ldv = ldv; a.off_v = off_v; a.ldo = ldo;
    a.H = H; a.heads_per_group = heads_per_group; a.d = d; a.dv = dv; a.dvx = dv + (ones ? 1 : 0);
    return a;
}

// Segments with fewer than qn_below new tokens (0: all), token by token.
extern "C" int locus_gated_scan(const float* q, int ldq, int off_q, const float* k, int ldk, int off_k, const float* v,
                                int ldv, int off_v, const float* keep, const float* take, float* state,
                                long long slot_stride, const int* state_slots, const int* seg_q0, const int* seg_qn,
                                int n_seg, float q_scale, float* out, int ldo, int H, int heads_per_group, int d, int dv,
                                int ones, int qn_below, cudaStream_t stream) {
    if (n_seg <= 0) return 0;
    const RecArgs a = rec_args(q, ldq, off_q, k, ldk, off_k, v, ldv, off_v, keep, take, state, slot_stride, state_slots,
                               seg_q0, seg_qn, q_scale, out, ldo, H, heads_per_group, d, dv, ones);
    if (!rec_args_ok(a, n_seg)) return LOCUS_ERR_UNSUPPORTED;
    const int col_groups = (a.dvx + REC_CW - 1) / REC_CW;
    const dim3 grid((H * col_groups + 3) / 4, n_seg);
    const int rpl = (d + 31) / 32;
#define SCAN(R) locus_launch(gated_scan_kernel<R>, grid, dim3(128), 0, stream, a, col_groups, qn_below)
    if (rpl <= 1) SCAN(1);
    else if (rpl <= 2) SCAN(2);
    else if (rpl <= 4) SCAN(4);
    else SCAN(8);
#undef SCAN
    return locus_launch_status();
}

// Segments with at least qn_from new tokens, chunk by chunk; longest_new: the most new tokens of a segment of the
// step (an upper bound will do: it sizes the first kernel's grid).
extern "C" int locus_gated_chunked(const float* q, int ldq, int off_q, const float* k, int ldk, int off_k, const float* v,
                                   int ldv, int off_v, const float* keep, const float* take, float* state,
                                   long long slot_stride, const int* state_slots, const int* seg_q0, const int* seg_qn,
                                   int n_seg, float q_scale, float* out, int ldo, int H, int heads_per_group, int d,
                                   int dv, int ones, int qn_from, int longest_new, cudaStream_t stream) {
    if (n_seg <= 0 || longest_new <= 0) return 0;
    const RecArgs a = rec_args(q, ldq, off_q, k, ldk, off_k, v, ldv, off_v, keep, take, state, slot_stride, state_slots,
                               seg_q0, seg_qn, q_scale, out, ldo, H, heads_per_group, d, dv, ones);
    if (!rec_args_ok(a, n_seg) || qn_from < 1) return LOCUS_ERR_UNSUPPORTED;
    const int d4 = (d + 3) & ~3, dvp = (a.dvx + 31) & ~31;
    const size_t smem1 = sizeof(float) * (2 * REC_CHUNK * (d4 + 4) + REC_CHUNK * (REC_CHUNK + 4) +
                                          static_cast<size_t>(REC_CHUNK) * dvp + REC_CHUNK * (REC_CHUNK + 1));
    if (smem1 > 200 * 1024) return LOCUS_ERR_UNSUPPORTED;
    if (smem1 > 48 * 1024 &&
        cudaFuncSetAttribute(gated_intra_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem1)) !=
            cudaSuccess)
        return LOCUS_ERR_UNSUPPORTED;
    locus_launch(gated_intra_kernel, dim3((longest_new + REC_CHUNK - 1) / REC_CHUNK, H, n_seg), dim3(256), smem1, stream, a,
                 qn_from);
    int cols = 32;
    while (cols > 8 && static_cast<long long>(H) * ((a.dvx + cols - 1) / cols) * n_seg < 148) cols >>= 1;
    const int col_groups = (a.dvx + cols - 1) / cols;
    const int lds = cols == 32 ? 32 : cols + cols / 4;
    const size_t smem2 = sizeof(float) * (2 * REC_CHUNK * (d4 + 4) + REC_CHUNK * cols + static_cast<size_t>(d4) * lds +
                                          10 * REC_CHUNK + 4);
    if (smem2 > 48 * 1024 &&
        cudaFuncSetAttribute(gated_inter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem2)) !=
            cudaSuccess)
        return LOCUS_ERR_UNSUPPORTED;
    locus_launch(gated_inter_kernel, dim3(H * col_groups, n_seg), dim3(256), smem2, stream, a, col_groups, cols, qn_from);
    return locus_launch_status();
}
