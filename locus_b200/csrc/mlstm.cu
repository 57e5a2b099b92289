// The gates and the output stage of a matrix memory with exponential gating (the recurrence itself is the gated
// linear recurrence of recurrence.cu, with the normaliser as one more column of the state).
//
// Per token and head, from the pre-activations zi and zf (float32 columns of the projection's rows):
//
//     i = cap * tanh(zi / cap),   f = logsigmoid(cap * tanh(zf / cap)),
//     m_t = max(f + m_(t-1), i),  keep_t = exp(f + m_(t-1) - m_t),  take_t = exp(i - m_t)
//
// m is carried in the request's state slot (it starts at 0 with the zeroed slot).  The recurrence then gives the
// numerator S_t^T q and, in its last column, n_t . q; the output stage divides by max(|n_t . q|, exp(-m_t)) + 1e-6,
// divides a head's row by its root mean square, and multiplies by a weight and by sigmoid(gate).
#include "common.cuh"

__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// One block per (head, segment), a tile of MG_TILE tokens at a time through shared memory: the pre-activations are
// turned into i and f by all threads, one thread walks the running maximum (additions and maxima only, operands in
// shared memory), all threads form keep and take.
#define MG_TILE 1024

__global__ void __launch_bounds__(256) mlstm_gates_kernel(const float* __restrict__ proj, int ld, int off_i, int off_f,
                                                          float cap, float* __restrict__ m_state, long long slot_stride,
                                                          const int* __restrict__ state_slots,
                                                          const int* __restrict__ seg_q0, const int* __restrict__ seg_qn,
                                                          float* __restrict__ keep, float* __restrict__ take,
                                                          float* __restrict__ m_out, int H) {
    __shared__ float s_i[MG_TILE], s_f[MG_TILE], s_m[MG_TILE + 1];
    pdl_entry();
    pdl_trigger();
    const int h = blockIdx.x, seg = blockIdx.y;
    const int q0 = seg_q0[seg], qn = seg_qn[seg];
    float* mp = m_state + static_cast<size_t>(state_slots[seg]) * slot_stride + h;
    if (threadIdx.x == 0) s_m[0] = *mp;
    for (int t0 = 0; t0 < qn; t0 += MG_TILE) {
        const int n = min(MG_TILE, qn - t0);
        for (int t = threadIdx.x; t < n; t += blockDim.x) {
            const size_t row = static_cast<size_t>(q0 + t0 + t);
            const float zi = proj[row * ld + off_i + h], zf = proj[row * ld + off_f + h];
            s_i[t] = cap * tanhf(zi / cap);
            s_f[t] = log_sigmoid(cap * tanhf(zf / cap));
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            float m = s_m[0];   // the maximum behind the tile before (or the slot's)
#pragma unroll 8
            for (int t = 0; t < n; ++t) {
                m = fmaxf(s_f[t] + m, s_i[t]);
                s_m[t + 1] = m;
            }
        }
        __syncthreads();
        for (int t = threadIdx.x; t < n; t += blockDim.x) {
            const size_t at = static_cast<size_t>(q0 + t0 + t) * H + h;
            const float m_prev = s_m[t], m = s_m[t + 1];
            keep[at] = expf(s_f[t] + m_prev - m);
            take[at] = expf(s_i[t] - m);
            m_out[at] = m;
        }
        __syncthreads();
        if (threadIdx.x == 0) s_m[0] = s_m[n];
        __syncthreads();
    }
    if (threadIdx.x == 0 && qn > 0) *mp = s_m[0];
}

// proj [T, ld] float32; m_state: the address of head 0's m in slot 0 (slots are slot_stride floats apart);
// keep, take, m_out [T, H] float32.
extern "C" int locus_mlstm_gates(const float* proj, int ld, int off_i, int off_f, float cap, float* m_state,
                                 long long slot_stride, const int* state_slots, const int* seg_q0, const int* seg_qn,
                                 int n_seg, float* keep, float* take, float* m_out, int H, cudaStream_t stream) {
    if (n_seg <= 0) return 0;
    if (H <= 0 || H > 65535 || n_seg > 65535 || !(cap > 0.f)) return LOCUS_ERR_UNSUPPORTED;
    locus_launch(mlstm_gates_kernel, dim3(H, n_seg), dim3(256), 0, stream, proj, ld, off_i, off_f, cap, m_state,
                 slot_stride, state_slots, seg_q0, seg_qn, keep, take, m_out, H);
    return locus_launch_status();
}

// A warp per (token, head).  o_raw [T, H * (dv + 1)]: a head's numerator and, behind it, n . q.
template <typename TW, typename TO>
__global__ void __launch_bounds__(256) mlstm_out_kernel(const float* __restrict__ o_raw, const float* __restrict__ m_t,
                                                        const float* __restrict__ proj, int ld, int off_g,
                                                        const TW* __restrict__ w, float eps, TO* __restrict__ out,
                                                        int n_units, int H, int dv) {
    pdl_entry();
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (unit >= n_units) return;
    const int t = unit / H, h = unit % H;
    const float* o = o_raw + (static_cast<size_t>(t) * H + h) * (dv + 1);
    const float den = fmaxf(fabsf(o[dv]), expf(-m_t[static_cast<size_t>(t) * H + h])) + 1e-6f;
    float ss = 0.f;
    for (int j = lane; j < dv; j += 32) {
        const float v = o[j] / den;
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / static_cast<float>(dv) + eps);
    const float* g = proj + static_cast<size_t>(t) * ld + off_g + h * dv;
    TO* dst = out + (static_cast<size_t>(t) * H + h) * dv;
    for (int j = lane; j < dv; j += 32)
        dst[j] = from_f<TO>(o[j] / den * scale * to_f(w[h * dv + j]) * (1.0f / (1.0f + expf(-g[j]))));
}

extern "C" int locus_mlstm_out(const float* o_raw, const float* m_t, const float* proj, int ld, int off_g, const void* w,
                               int w_dt, float eps, void* out, int out_dt, int T, int H, int dv, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || dv <= 0) return LOCUS_ERR_UNSUPPORTED;
    const long long units = static_cast<long long>(T) * H;
    if (units > 0x7fffffffLL) return LOCUS_ERR_UNSUPPORTED;
    const int blocks = static_cast<int>((units + 7) / 8), n = static_cast<int>(units);
#define OUT(TW, TO)                                                                                                  \
    locus_launch(mlstm_out_kernel<TW, TO>, blocks, 256, 0, stream, o_raw, m_t, proj, ld, off_g,                      \
                 static_cast<const TW*>(w), eps, static_cast<TO*>(out), n, H, dv)
    if (w_dt == LOCUS_DT_BF16 && out_dt == LOCUS_DT_BF16) OUT(bf16, bf16);
    else if (w_dt == LOCUS_DT_F32 && out_dt == LOCUS_DT_F32) OUT(float, float);
    else if (w_dt == LOCUS_DT_BF16 && out_dt == LOCUS_DT_F32) OUT(bf16, float);
    else if (w_dt == LOCUS_DT_F32 && out_dt == LOCUS_DT_BF16) OUT(float, bf16);
    else return LOCUS_ERR_UNSUPPORTED;
#undef OUT
    return locus_launch_status();
}
