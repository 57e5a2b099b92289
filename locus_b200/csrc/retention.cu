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
//   retention_gate_norm  out[t, h, :] = o[t, h, :] / rms(o[t, h, :]) * silu(g[t, h, :])   (a warp per row and head)
#include "common.cuh"

#define RET_CW 4

template <int RPL>
__global__ void __launch_bounds__(128) retention_scan_kernel(
    const float* __restrict__ qkvg, int ld, float* __restrict__ state, const int* __restrict__ state_slots,
    const int* __restrict__ seg_q0, const int* __restrict__ seg_qn, const float* __restrict__ decay, float k_scale,
    float* __restrict__ o_raw, int H, int d, int dv, int col_groups) {
    pdl_entry();
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.x * 4 + (threadIdx.x >> 5);  // (head, column group)
    const int seg = blockIdx.y;
    if (unit >= H * col_groups) return;
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
// o_raw [T, H * dv] float32.  d <= 256.
extern "C" int locus_retention_scan(const float* qkvg, int ld, float* state, const int* state_slots,
                                    const int* seg_q0, const int* seg_qn, int n_seg, const float* decay,
                                    float k_scale, float* o_raw, int H, int d, int dv, cudaStream_t stream) {
    if (n_seg <= 0) return 0;
    if (H <= 0 || d <= 0 || d > 256 || dv <= 0 || n_seg > 65535 || ld < 2 * H * d + 2 * H * dv) return LOCUS_ERR_UNSUPPORTED;
    const int col_groups = (dv + RET_CW - 1) / RET_CW;
    const dim3 grid((H * col_groups + 3) / 4, n_seg);
    const int rpl = (d + 31) / 32;
#define SCAN(R)                                                                                                 \
    locus_launch(retention_scan_kernel<R>, grid, dim3(128), 0, stream, qkvg, ld, state, state_slots, seg_q0,    \
                 seg_qn, decay, k_scale, o_raw, H, d, dv, col_groups)
    if (rpl <= 1) SCAN(1);
    else if (rpl <= 2) SCAN(2);
    else if (rpl <= 4) SCAN(4);
    else SCAN(8);
#undef SCAN
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
