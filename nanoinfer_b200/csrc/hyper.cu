// Hyper-connections: instead of one residual stream a layer keeps S copies x_0 .. x_{S-1} (all equal to the
// embedding's output at the start).  A sublayer reads u = sum_s in[s] x_s through a norm, and its result y goes back
// into all copies at once:   x_t <- sum_s mix[s, t] x_s + out[t] * y   (mix indexed [from, to]).
// With a gated residual, y is first multiplied element by element by sigmoid(gate), the gate's logits coming from
// a product of the sublayer's own input.
//
// hyper_update does, for a row, in ONE pass over the row: the gate, the new copies, y zeroed again for the next
// sublayer, the next sublayer's input  xn = u' / sqrt(mean(u'^2) + eps) * w_next  with u' = sum_s in_next[s] x_s
// (in the engine's dtype), and, where asked for, the sum of the copies (what leaves the last layer).  Everything is
// 32-bit; a block owns a row and keeps u' in shared memory between the pass that makes it and the one that scales it.
// hyper_enter makes the S copies from the one stream and the first sublayer's input.
#include "api.h"
#include "common.cuh"

namespace nib {

constexpr int HYPER_MAX_STREAMS = 8;

template <typename OutT>
__global__ void __launch_bounds__(256)
hyper_enter_kernel(const float* x, float* streams, long long stream_stride, int S, const float* __restrict__ in_w,
                   const float* __restrict__ w_next, float eps, OutT* xn, int C) {
  pdl_trigger();
  extern __shared__ float u_row[];
  __shared__ float scratch[32];
  const size_t t = blockIdx.x;
  float total_in = 0.0f;
  for (int s = 0; s < S; ++s) total_in += in_w[s];
  pdl_wait();
  float ss = 0.0f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float v = x[t * C + c];
    for (int s = 0; s < S; ++s) streams[(size_t)s * stream_stride + t * C + c] = v;
    const float u = total_in * v;
    u_row[c] = u;
    ss += u * u;
  }
  const float r = 1.0f / sqrtf(block_sum(ss, scratch) / (float)C + eps);
  for (int c = threadIdx.x; c < C; c += blockDim.x) xn[t * C + c] = from_float<OutT>(u_row[c] * r * w_next[c]);
}

template <typename OutT>
__global__ void __launch_bounds__(256)
hyper_update_kernel(float* streams, long long stream_stride, int S, float* y, const float* gate, int ldg,
                    const float* __restrict__ mix, const float* __restrict__ out_w, const float* __restrict__ in_next,
                    const float* __restrict__ w_next, float eps, OutT* xn, float* total, int C) {
  pdl_trigger();
  extern __shared__ float u_row[];
  __shared__ float scratch[32];
  __shared__ float m_sh[HYPER_MAX_STREAMS * HYPER_MAX_STREAMS], o_sh[HYPER_MAX_STREAMS], i_sh[HYPER_MAX_STREAMS];
  const size_t t = blockIdx.x;
  if (threadIdx.x < S * S) m_sh[threadIdx.x] = mix[threadIdx.x];
  if (threadIdx.x < S) {
    o_sh[threadIdx.x] = out_w[threadIdx.x];
    i_sh[threadIdx.x] = in_next ? in_next[threadIdx.x] : 0.0f;
  }
  __syncthreads();
  pdl_wait();
  float ss = 0.0f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float r = y[t * C + c];
    if (gate != nullptr) r *= 1.0f / (1.0f + expf(-gate[t * ldg + c]));
    y[t * C + c] = 0.0f;
    float old[HYPER_MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < HYPER_MAX_STREAMS; ++s) old[s] = s < S ? streams[(size_t)s * stream_stride + t * C + c] : 0.0f;
    float u = 0.0f, sum = 0.0f;
#pragma unroll
    for (int to = 0; to < HYPER_MAX_STREAMS; ++to) {
      if (to < S) {
        float v = 0.0f;
#pragma unroll
        for (int s = 0; s < HYPER_MAX_STREAMS; ++s)
          if (s < S) v = fmaf(m_sh[s * S + to], old[s], v);
        v = fmaf(o_sh[to], r, v);
        streams[(size_t)to * stream_stride + t * C + c] = v;
        u = fmaf(i_sh[to], v, u);
        sum += v;
      }
    }
    if (total != nullptr) total[t * C + c] = sum;
    if (xn != nullptr) {
      u_row[c] = u;
      ss += u * u;
    }
  }
  if (xn == nullptr) return;
  const float rinv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)C + eps);
  for (int c = threadIdx.x; c < C; c += blockDim.x) xn[t * C + c] = from_float<OutT>(u_row[c] * rinv * w_next[c]);
}

}  // namespace nib

using namespace nib;

// x [T, C] float -> streams [S][T, C] (the copies lie stream_stride floats apart), xn [T, C] in `dtype`.
extern "C" int nib_hyper_enter(int dtype, const float* x, float* streams, long long stream_stride, int S,
                               const float* in_w, const float* w_next, float eps, void* xn, int T, int C,
                               cudaStream_t stream) {
  if (T <= 0) return 0;
  if (S <= 0 || S > HYPER_MAX_STREAMS || C <= 0 || (size_t)C * sizeof(float) > 200 * 1024) return NIB_ERR_UNSUPPORTED_SIZE;
  const size_t smem = (size_t)C * sizeof(float);
  if (dtype == DT_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(hyper_enter_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(hyper_enter_kernel<float>, dim3(T), dim3(256), smem, stream, x, streams, stream_stride, S, in_w, w_next,
               eps, (float*)xn, C);
  } else if (dtype == DT_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(hyper_enter_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(hyper_enter_kernel<bf16>, dim3(T), dim3(256), smem, stream, x, streams, stream_stride, S, in_w, w_next,
               eps, (bf16*)xn, C);
  } else {
    return NIB_ERR_BAD_ARGUMENT;
  }
  NIB_LAUNCH_CHECK();
}

// y [T, C] float is consumed and zeroed; gate (may be null) [T, ldg] float holds the gate's logits; mix [S, S]
// ([from, to]), out_w [S]; with xn: in_next [S] and w_next [C] make the next sublayer's input; total (may be null)
// receives the sum of the new copies.
extern "C" int nib_hyper_update(int dtype, float* streams, long long stream_stride, int S, float* y, const float* gate,
                                int ldg, const float* mix, const float* out_w, const float* in_next,
                                const float* w_next, float eps, void* xn, float* total, int T, int C,
                                cudaStream_t stream) {
  if (T <= 0) return 0;
  if (S <= 0 || S > HYPER_MAX_STREAMS || C <= 0 || (size_t)C * sizeof(float) > 200 * 1024) return NIB_ERR_UNSUPPORTED_SIZE;
  if (xn != nullptr && (in_next == nullptr || w_next == nullptr)) return NIB_ERR_BAD_ARGUMENT;
  const size_t smem = (size_t)C * sizeof(float);
  if (dtype == DT_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(hyper_update_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(hyper_update_kernel<float>, dim3(T), dim3(256), smem, stream, streams, stream_stride, S, y, gate, ldg, mix,
               out_w, in_next, w_next, eps, (float*)xn, total, C);
  } else if (dtype == DT_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(hyper_update_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(hyper_update_kernel<bf16>, dim3(T), dim3(256), smem, stream, streams, stream_stride, S, y, gate, ldg, mix,
               out_w, in_next, w_next, eps, (bf16*)xn, total, C);
  } else {
    return NIB_ERR_BAD_ARGUMENT;
  }
  NIB_LAUNCH_CHECK();
}
