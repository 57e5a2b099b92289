// The pieces of a selective state-space mixer around its recurrence (which is the gated linear recurrence of
// recurrence.cu: keep = exp(-exp(A_log) dt), take = dt, k = B, q = C, v = x).
//
//   ssm_conv        the short causal convolution per channel over [x | B | C], its bias and silu; a portion's first
//                   tokens read the inputs of the tokens before it from the request's state slot (zeros at a
//                   request's start: the slot is zeroed).  The same launch forms dt = softplus(dt_raw + dt_bias), keep
//                   and take for every (token, head).
//   ssm_conv_state  afterwards: the slot's last taps - 1 inputs move on by the portion's tokens.
//   ssm_out         (y + D x) * silu(z), divided by the root mean square of each of `parts` equal parts of the row,
//                   times a weight.
// All arithmetic is float32; the projection's rows arrive as float32.
#include "common.cuh"

#define SSM_MAX_TAPS 16

__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }

__global__ void __launch_bounds__(256) ssm_conv_kernel(
    const float* __restrict__ proj, int ld, int off_xbc, int off_dt, const void* __restrict__ cw, const void* __restrict__ cb,
    int w_dt, const void* __restrict__ dt_bias, const void* __restrict__ a_log, int p_dt,
    const float* __restrict__ conv_state, long long slot_stride, const int* __restrict__ state_slots,
    const int* __restrict__ seg_q0, const int* __restrict__ seg_qn, float* __restrict__ act, float* __restrict__ keep,
    float* __restrict__ take, int channels, int taps, int H) {
    pdl_entry();
    pdl_trigger();
    const int seg = blockIdx.z, t = blockIdx.y;
    const int qn = seg_qn[seg];
    if (t >= qn) return;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const size_t row = static_cast<size_t>(seg_q0[seg] + t);
    if (c < channels) {
        const float* old = conv_state + static_cast<size_t>(state_slots[seg]) * slot_stride + static_cast<size_t>(c) * (taps - 1);
        float acc = ld_dyn(cb, w_dt, c);
        for (int j = 0; j < taps; ++j) {
            const int p = t - (taps - 1) + j;   // the input's place within the portion; negative: before it
            const float x = p >= 0 ? proj[(row - (t - p)) * ld + off_xbc + c] : old[taps - 1 + p];
            acc = fmaf(ld_dyn(cw, w_dt, static_cast<size_t>(c) * taps + j), x, acc);
        }
        act[row * channels + c] = silu_f(acc);
    }
    if (c < H) {
        const float dt = softplus_f(proj[row * ld + off_dt + c] + ld_dyn(dt_bias, p_dt, c));
        keep[row * H + c] = expf(-expf(ld_dyn(a_log, p_dt, c)) * dt);
        take[row * H + c] = dt;
    }
}

__global__ void __launch_bounds__(256) ssm_conv_state_kernel(const float* __restrict__ proj, int ld, int off_xbc,
                                                             float* __restrict__ conv_state, long long slot_stride,
                                                             const int* __restrict__ state_slots,
                                                             const int* __restrict__ seg_q0,
                                                             const int* __restrict__ seg_qn, int channels, int taps) {
    pdl_entry();
    pdl_trigger();
    const int seg = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int qn = seg_qn[seg], q0 = seg_q0[seg], keep_n = taps - 1;
    float* st = conv_state + static_cast<size_t>(state_slots[seg]) * slot_stride + static_cast<size_t>(c) * keep_n;
    float nv[SSM_MAX_TAPS];
    for (int j = 0; j < keep_n; ++j) {
        const int p = qn - keep_n + j;
        nv[j] = p >= 0 ? proj[static_cast<size_t>(q0 + p) * ld + off_xbc + c] : st[j + qn];
    }
    for (int j = 0; j < keep_n; ++j) st[j] = nv[j];
}

// proj [T, ld] float32 with the columns [.. | x B C at off_xbc | dt at off_dt]; conv weights [channels, taps] and bias
// [channels] (element type w_dt), dt_bias and A_log [H] (element type p_dt); conv_state: the address of the
// convolution's part of slot 0 ([channels, taps - 1] float32, slots slot_stride floats apart); act [T, channels],
// keep and take [T, H] float32.  longest_new: the most new tokens of a segment (an upper bound will do).
extern "C" int locus_ssm_conv(const float* proj, int ld, int off_xbc, int off_dt, const void* cw, const void* cb, int w_dt,
                              const void* dt_bias, const void* a_log, int p_dt, float* conv_state, long long slot_stride,
                              const int* state_slots, const int* seg_q0, const int* seg_qn, int n_seg, int longest_new,
                              float* act, float* keep, float* take, int channels, int taps, int H, cudaStream_t stream) {
    if (n_seg <= 0 || longest_new <= 0) return 0;
    if (channels <= 0 || H <= 0 || taps < 1 || taps > SSM_MAX_TAPS || n_seg > 65535 || longest_new > 65535)
        return LOCUS_ERR_UNSUPPORTED;
    const int wide = channels > H ? channels : H;
    locus_launch(ssm_conv_kernel, dim3((wide + 255) / 256, longest_new, n_seg), dim3(256), 0, stream, proj, ld, off_xbc,
                 off_dt, cw, cb, w_dt, dt_bias, a_log, p_dt, static_cast<const float*>(conv_state), slot_stride,
                 state_slots, seg_q0, seg_qn, act, keep, take, channels, taps, H);
    if (taps > 1)
        locus_launch(ssm_conv_state_kernel, dim3((channels + 255) / 256, n_seg), dim3(256), 0, stream, proj, ld, off_xbc,
                     conv_state, slot_stride, state_slots, seg_q0, seg_qn, channels, taps);
    return locus_launch_status();
}

// A group of GT threads per (token, part of the row): a warp for narrow parts, a block of 256 for wide ones.
template <typename TO, int GT>
__global__ void __launch_bounds__(256) ssm_out_kernel(const float* __restrict__ y, const float* __restrict__ act,
                                                      int channels, const float* __restrict__ proj, int ld, int off_z,
                                                      const void* __restrict__ dskip, int p_dt, const void* __restrict__ w,
                                                      int w_dt, float eps, TO* __restrict__ out, int n_units, int parts,
                                                      int inner, int dv) {
    __shared__ float part_sum[8];
    pdl_entry();
    pdl_trigger();
    const int lane = threadIdx.x % GT;
    const int unit = blockIdx.x * (256 / GT) + threadIdx.x / GT;
    if (unit >= n_units) return;   // (a whole block at once when GT is 256)
    const int t = unit / parts, part = unit % parts, width = inner / parts, e0 = part * width;
    const float* yr = y + static_cast<size_t>(t) * inner;
    const float* xr = act + static_cast<size_t>(t) * channels;
    const float* zr = proj + static_cast<size_t>(t) * ld + off_z;
    float ss = 0.f;
    for (int j = lane; j < width; j += GT) {
        const int e = e0 + j;
        const float v = fmaf(ld_dyn(dskip, p_dt, e / dv), xr[e], yr[e]) * silu_f(zr[e]);
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    if (GT == 256) {
        if ((threadIdx.x & 31) == 0) part_sum[threadIdx.x >> 5] = ss;
        __syncthreads();
        ss = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) ss += part_sum[k];
    }
    const float scale = 1.0f / sqrtf(ss / static_cast<float>(width) + eps);
    TO* dst = out + static_cast<size_t>(t) * inner;
    for (int j = lane; j < width; j += GT) {
        const int e = e0 + j;
        const float v = fmaf(ld_dyn(dskip, p_dt, e / dv), xr[e], yr[e]) * silu_f(zr[e]);
        dst[e] = from_f<TO>(v * scale * ld_dyn(w, w_dt, e));
    }
}

// y [T, inner] float32 (the recurrence's output), act [T, channels] (x in its first `inner` columns), z at off_z of
// proj's rows, dskip [inner / dv] (element type p_dt), w [inner] (element type w_dt); out [T, inner].
extern "C" int locus_ssm_out(const float* y, const float* act, int channels, const float* proj, int ld, int off_z,
                             const void* dskip, int p_dt, const void* w, int w_dt, float eps, void* out, int out_dt, int T,
                             int parts, int inner, int dv, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (parts <= 0 || inner <= 0 || inner % parts || dv <= 0 || inner % dv) return LOCUS_ERR_UNSUPPORTED;
    const long long units = static_cast<long long>(T) * parts;
    if (units > 0x7fffffffLL) return LOCUS_ERR_UNSUPPORTED;
    const bool wide = inner / parts >= 1024;
    const int n = static_cast<int>(units), blocks = wide ? n : static_cast<int>((units + 7) / 8);
#define SSM_OUT(TO, GT)                                                                                              \
    locus_launch(ssm_out_kernel<TO, GT>, blocks, 256, 0, stream, y, act, channels, proj, ld, off_z, dskip, p_dt, w, w_dt, \
                 eps, static_cast<TO*>(out), n, parts, inner, dv)
    if (out_dt == LOCUS_DT_BF16) {
        if (wide) SSM_OUT(bf16, 256); else SSM_OUT(bf16, 32);
    } else if (out_dt == LOCUS_DT_F32) {
        if (wide) SSM_OUT(float, 256); else SSM_OUT(float, 32);
    } else {
        return LOCUS_ERR_UNSUPPORTED;
    }
#undef SSM_OUT
    return locus_launch_status();
}
