// Kernels on the 32-bit residual stream for layers that normalise AFTER the sum:
//   x <- norm(alpha * x + sublayer(x))
// and for models that hand each layer a weighted average of all earlier layers' results.
//
// The stream is kept pre-scaled: a sublayer's last product adds into alpha * x, which the kernel
// before it has left in place together with the sublayer's input (x itself, in the engine's dtype).
//   stream_enter : xn = cast(x); level0 = x (optional); x = alpha * x
//   post_norm    : y = x / sqrt(mean(x^2) + eps) * w;
//                  with levels: level[n-1] = y; z = sum_j mix[j] * level[j]   (j ascending), else z = y;
//                  xn = cast(z) (optional); x = alpha_next * z
//   rmsnorm      : out[r] = x[rows[r]] / sqrt(mean + eps) * w   (the model's last norm, wanted rows only)
//   act          : tanh, or xIELU with its two numbers p, q read from the device:
//                  z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2
// and for layers that normalise a sublayer's output before the sum as well as its input:
//   add_norm     : x += y / sqrt(mean(y^2) + eps) * w_out;  y = 0 (the next sublayer adds its products into it);
//                  xn = cast(x / sqrt(mean(x^2) + eps) * w_next)   (optional: the next sublayer's input)
//   glu          : out[t, f] = act(pre[t, 2f]) * pre[t, 2f + 1] (* sigmoid(pre[t, row_gate]) if asked for)
// Statistics, sums and the activation's arithmetic are 32-bit.
#include <cstdint>

#include "api.h"
#include "common.cuh"

namespace nib {

__device__ __forceinline__ void store4(float* p, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(bf16* p, float a, float b, float c, float d) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&lo);
  u.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = u;
}

template <typename OutT>
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const float* x, const int* __restrict__ rows, const float* __restrict__ w, OutT* out, int C,
               float eps) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ float smem[];
  float* row = smem;
  float* scratch = smem + C;
  const int r = blockIdx.x;
  const float* src = x + (size_t)(rows ? rows[r] : r) * C;
  float q = 0.0f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float v = src[c];
    row[c] = v;
    q += v * v;
  }
  const float rstd = 1.0f / sqrtf(block_sum(q, scratch) / (float)C + eps);
  OutT* o = out + (size_t)r * C;
  for (int c = threadIdx.x; c < C; c += blockDim.x) o[c] = from_float<OutT>(row[c] * rstd * w[c]);
}

template <typename OutT>
__global__ void __launch_bounds__(256)
stream_enter_kernel(float* x, OutT* xn, float* level0, float alpha, size_t n) {
  pdl_trigger();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float v = x[i];
  xn[i] = from_float<OutT>(v);
  if (level0 != nullptr) level0[i] = v;
  x[i] = alpha * v;
}

template <typename OutT>
__global__ void __launch_bounds__(256)
post_norm_kernel(float* x, const float* __restrict__ w, float eps, float* levels, long long level_stride,
                 int n_levels, const float* __restrict__ mix, OutT* xn, float alpha_next, int C) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ float smem[];
  float* row = smem;
  float* scratch = smem + C;
  const size_t base = (size_t)blockIdx.x * C;
  float q = 0.0f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float v = x[base + c];
    row[c] = v;
    q += v * v;
  }
  const float rstd = 1.0f / sqrtf(block_sum(q, scratch) / (float)C + eps);
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float y = row[c] * rstd * w[c];
    float z = y;
    if (levels != nullptr) {
      levels[(size_t)(n_levels - 1) * level_stride + base + c] = y;
      z = 0.0f;
      for (int j = 0; j + 1 < n_levels; ++j) z += mix[j] * levels[(size_t)j * level_stride + base + c];
      z += mix[n_levels - 1] * y;
    }
    if (xn != nullptr) xn[base + c] = from_float<OutT>(z);
    x[base + c] = alpha_next * z;
  }
}

// One kernel between two sublayers: the norm of what the last one made, the sum, and the norm that the next one reads.
template <typename OutT>
__global__ void __launch_bounds__(256)
add_norm_kernel(float* x, float* y, const float* __restrict__ w_out, const float* __restrict__ w_next, float eps,
                OutT* xn, int C) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ float smem[];
  float* row = smem;
  float* scratch = smem + C;
  const size_t base = (size_t)blockIdx.x * C;
  float q = 0.0f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float v = y[base + c];
    y[base + c] = 0.0f;
    row[c] = v;
    q += v * v;
  }
  const float rstd = 1.0f / sqrtf(block_sum(q, scratch) / (float)C + eps);
  float q2 = 0.0f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float v = x[base + c] + row[c] * rstd * w_out[c];
    x[base + c] = v;
    row[c] = v;
    q2 += v * v;
  }
  if (xn == nullptr) return;
  if (w_next == nullptr) {   // the next sublayer reads the stream itself
    for (int c = threadIdx.x; c < C; c += blockDim.x) xn[base + c] = from_float<OutT>(row[c]);
    return;
  }
  const float rstd2 = 1.0f / sqrtf(block_sum(q2, scratch) / (float)C + eps);
  for (int c = threadIdx.x; c < C; c += blockDim.x) xn[base + c] = from_float<OutT>(row[c] * rstd2 * w_next[c]);
}

// The same with a warp a row and the row in registers (widths that are multiples of 4 up to 128 * NV): no shared
// memory, no block barrier; eight rows a block.  The sums run in the order lane-local values, then the warp's
// butterfly, whatever the number of rows: a row's bits do not depend on the step's size.
template <typename OutT, int NV>
__global__ void __launch_bounds__(256)
add_norm_rows_kernel(float* x, float* y, const float* __restrict__ w_out, const float* __restrict__ w_next, float eps,
                     OutT* xn, int n_rows, int C) {
  pdl_trigger();
  const int lane = threadIdx.x & 31, row = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int n4 = C >> 2;                    // 16-byte pieces of a row; lane owns pieces lane, lane + 32, ...
  float4 wo[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i)
    if (lane + 32 * i < n4) wo[i] = reinterpret_cast<const float4*>(w_out)[lane + 32 * i];
  pdl_wait();
  if (row >= n_rows) return;
  float4* yr = reinterpret_cast<float4*>(y + (size_t)row * C);
  float4* xr = reinterpret_cast<float4*>(x + (size_t)row * C);
  float4 v[NV];
  float q = 0.0f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    if (lane + 32 * i < n4) {
      v[i] = yr[lane + 32 * i];
      yr[lane + 32 * i] = make_float4(0.f, 0.f, 0.f, 0.f);
      q += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    }
  }
  const float rstd = 1.0f / sqrtf(warp_sum(q) / (float)C + eps);
  float q2 = 0.0f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    if (lane + 32 * i < n4) {
      const float4 a = xr[lane + 32 * i];
      v[i] = make_float4(a.x + v[i].x * rstd * wo[i].x, a.y + v[i].y * rstd * wo[i].y, a.z + v[i].z * rstd * wo[i].z,
                         a.w + v[i].w * rstd * wo[i].w);
      xr[lane + 32 * i] = v[i];
      q2 += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    }
  }
  if (xn == nullptr) return;
  OutT* o = xn + (size_t)row * C;
  if (w_next == nullptr) {   // the next sublayer reads the stream itself
#pragma unroll
    for (int i = 0; i < NV; ++i)
      if (lane + 32 * i < n4) store4(o + 4 * (lane + 32 * i), v[i].x, v[i].y, v[i].z, v[i].w);
    return;
  }
  const float rstd2 = 1.0f / sqrtf(warp_sum(q2) / (float)C + eps);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    if (lane + 32 * i < n4) {
      const float4 wn = reinterpret_cast<const float4*>(w_next)[lane + 32 * i];
      store4(o + 4 * (lane + 32 * i), v[i].x * rstd2 * wn.x, v[i].y * rstd2 * wn.y, v[i].z * rstd2 * wn.z, v[i].w * rstd2 * wn.w);
    }
  }
}

// pre [T, ld]: pairs (gate, value) side by side, F of them; row_gate >= 0: one more column whose sigmoid scales the row
template <typename InT, typename OutT>
__global__ void __launch_bounds__(256)
glu_kernel(const InT* pre, int ld, OutT* out, int ldo, int n_rows, int F, int act, int row_gate) {
  pdl_trigger();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)n_rows * F) return;
  const int t = (int)(i / F), f = (int)(i % F);
  const InT* p = pre + (size_t)t * ld;
  float v = apply_act(to_float(p[2 * f]), act) * to_float(p[2 * f + 1]);
  if (row_gate >= 0) v *= 1.0f / (1.0f + expf(-to_float(p[row_gate])));
  out[(size_t)t * ldo + f] = from_float<OutT>(v);
}

enum : int { UNARY_TANH = 1, UNARY_XIELU = 2, UNARY_SOFTCAP = 3, UNARY_SCALE = 4 };   // softcap: prm[0] tanh(z / prm[0]); scale: prm[0] z

__device__ __forceinline__ float softplus_f(float v) { return v > 20.0f ? v : log1pf(expf(v)); }

template <typename InT, typename OutT>
__global__ void __launch_bounds__(256)
unary_kernel(const InT* in, int ld_in, OutT* out, int ld_out, int n_rows, int n_cols, int kind,
             const float* __restrict__ prm) {
  pdl_trigger();
  float sp = 0.0f, sq = 0.0f;
  if (kind == UNARY_XIELU) {
    sp = softplus_f(prm[0]);
    sq = 0.5f + softplus_f(prm[1]);
  }
  if (kind == UNARY_SOFTCAP || kind == UNARY_SCALE) sp = prm[0];
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)n_rows * n_cols) return;
  const int r = (int)(i / n_cols), c = (int)(i % n_cols);
  const float z = to_float(in[(size_t)r * ld_in + c]);
  float y;
  if (kind == UNARY_TANH)
    y = tanhf(z);
  else if (kind == UNARY_SOFTCAP)
    y = sp * tanhf(z / sp);
  else if (kind == UNARY_SCALE)
    y = sp * z;
  else
    y = z > 0.0f ? sp * z * z + 0.5f * z : sq * (expm1f(z) - z) + 0.5f * z;
  out[(size_t)r * ld_out + c] = from_float<OutT>(y);
}

}  // namespace nib

using namespace nib;

extern "C" int nib_rmsnorm(int out_dtype, const float* x, const int* rows, const float* w, void* out, int n_rows,
                           int C, float eps, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (C <= 0 || C > 48000) return NIB_ERR_UNSUPPORTED_SIZE;
  const size_t smem = (size_t)(C + 32) * sizeof(float);
  const int threads = C >= 1024 ? 256 : 128;
  if (out_dtype == DT_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), smem, stream, x, rows, w, (float*)out, C, eps);
  } else if (out_dtype == DT_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(rmsnorm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(rmsnorm_kernel<bf16>, dim3(n_rows), dim3(threads), smem, stream, x, rows, w, (bf16*)out, C, eps);
  } else {
    return NIB_ERR_BAD_ARGUMENT;
  }
  NIB_LAUNCH_CHECK();
}

extern "C" int nib_stream_enter(int out_dtype, float* x, void* xn, float* level0, float alpha, int n_rows, int C,
                                cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  const size_t n = (size_t)n_rows * C;
  const dim3 grid((unsigned)((n + 255) / 256));
  if (out_dtype == DT_F32)
    launch_pdl(stream_enter_kernel<float>, grid, dim3(256), 0, stream, x, (float*)xn, level0, alpha, n);
  else if (out_dtype == DT_BF16)
    launch_pdl(stream_enter_kernel<bf16>, grid, dim3(256), 0, stream, x, (bf16*)xn, level0, alpha, n);
  else
    return NIB_ERR_BAD_ARGUMENT;
  NIB_LAUNCH_CHECK();
}

extern "C" int nib_post_norm(int out_dtype, float* x, const float* w, float eps, float* levels,
                             long long level_stride, int n_levels, const float* mix, void* xn, float alpha_next,
                             int n_rows, int C, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (C <= 0 || C > 48000) return NIB_ERR_UNSUPPORTED_SIZE;
  if (levels != nullptr && (n_levels < 1 || mix == nullptr)) return NIB_ERR_BAD_ARGUMENT;
  const size_t smem = (size_t)(C + 32) * sizeof(float);
  const int threads = C >= 1024 ? 256 : 128;
  if (out_dtype == DT_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(post_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(post_norm_kernel<float>, dim3(n_rows), dim3(threads), smem, stream, x, w, eps, levels, level_stride,
               n_levels, mix, (float*)xn, alpha_next, C);
  } else if (out_dtype == DT_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(post_norm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(post_norm_kernel<bf16>, dim3(n_rows), dim3(threads), smem, stream, x, w, eps, levels, level_stride,
               n_levels, mix, (bf16*)xn, alpha_next, C);
  } else {
    return NIB_ERR_BAD_ARGUMENT;
  }
  NIB_LAUNCH_CHECK();
}

extern "C" int nib_add_norm(int out_dtype, float* x, float* y, const float* w_out, const float* w_next, float eps,
                            void* xn, int n_rows, int C, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (C <= 0 || C > 48000) return NIB_ERR_UNSUPPORTED_SIZE;
  if (w_next != nullptr && xn == nullptr) return NIB_ERR_BAD_ARGUMENT;
  const bool vec = (C & 3) == 0 && C <= 2048 &&
                   (((uintptr_t)x | (uintptr_t)y | (uintptr_t)w_out | (uintptr_t)w_next | (uintptr_t)xn) & 15) == 0;
  if (vec) {   // whatever the number of rows
    const dim3 grid((n_rows + 7) / 8);
#define NIB_AN(T, NV) launch_pdl(add_norm_rows_kernel<T, NV>, grid, dim3(256), 0, stream, x, y, w_out, w_next, eps, (T*)xn, n_rows, C)
    if (out_dtype == DT_F32) { if (C <= 1024) NIB_AN(float, 8); else NIB_AN(float, 16); }
    else if (out_dtype == DT_BF16) { if (C <= 1024) NIB_AN(bf16, 8); else NIB_AN(bf16, 16); }
    else return NIB_ERR_BAD_ARGUMENT;
#undef NIB_AN
    NIB_LAUNCH_CHECK();
  }
  const size_t smem = (size_t)(C + 32) * sizeof(float);
  const int threads = C >= 1024 ? 256 : 128;
  if (out_dtype == DT_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(add_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(add_norm_kernel<float>, dim3(n_rows), dim3(threads), smem, stream, x, y, w_out, w_next, eps, (float*)xn, C);
  } else if (out_dtype == DT_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(add_norm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(add_norm_kernel<bf16>, dim3(n_rows), dim3(threads), smem, stream, x, y, w_out, w_next, eps, (bf16*)xn, C);
  } else {
    return NIB_ERR_BAD_ARGUMENT;
  }
  NIB_LAUNCH_CHECK();
}

// act: an activation code of the linear epilogues, applied to the gate of each pair.
extern "C" int nib_glu(int in_dtype, int out_dtype, const void* pre, int ld, void* out, int ldo, int n_rows, int F,
                       int act, int row_gate, cudaStream_t stream) {
  if (n_rows <= 0 || F <= 0) return 0;
  const size_t n = (size_t)n_rows * F;
  const dim3 grid((unsigned)((n + 255) / 256));
  if (in_dtype == DT_F32 && out_dtype == DT_F32)
    launch_pdl(glu_kernel<float, float>, grid, dim3(256), 0, stream, (const float*)pre, ld, (float*)out, ldo, n_rows, F,
               act, row_gate);
  else if (in_dtype == DT_F32 && out_dtype == DT_BF16)
    launch_pdl(glu_kernel<float, bf16>, grid, dim3(256), 0, stream, (const float*)pre, ld, (bf16*)out, ldo, n_rows, F,
               act, row_gate);
  else if (in_dtype == DT_BF16 && out_dtype == DT_BF16)
    launch_pdl(glu_kernel<bf16, bf16>, grid, dim3(256), 0, stream, (const bf16*)pre, ld, (bf16*)out, ldo, n_rows, F,
               act, row_gate);
  else
    return NIB_ERR_BAD_ARGUMENT;
  NIB_LAUNCH_CHECK();
}

// kind 1: tanh; kind 2: xIELU with prm = {p, q} on the device.  in and out may be the same buffer.
extern "C" int nib_unary(int in_dtype, int out_dtype, const void* in, int ld_in, void* out, int ld_out, int n_rows,
                         int n_cols, int kind, const float* prm, cudaStream_t stream) {
  if (n_rows <= 0 || n_cols <= 0) return 0;
  if (kind != UNARY_TANH && kind != UNARY_XIELU && kind != UNARY_SOFTCAP && kind != UNARY_SCALE) return NIB_ERR_BAD_ARGUMENT;
  if (kind != UNARY_TANH && prm == nullptr) return NIB_ERR_BAD_ARGUMENT;
  const size_t n = (size_t)n_rows * n_cols;
  const dim3 grid((unsigned)((n + 255) / 256));
  if (in_dtype == DT_F32 && out_dtype == DT_F32)
    launch_pdl(unary_kernel<float, float>, grid, dim3(256), 0, stream, (const float*)in, ld_in, (float*)out, ld_out,
               n_rows, n_cols, kind, prm);
  else if (in_dtype == DT_F32 && out_dtype == DT_BF16)
    launch_pdl(unary_kernel<float, bf16>, grid, dim3(256), 0, stream, (const float*)in, ld_in, (bf16*)out, ld_out,
               n_rows, n_cols, kind, prm);
  else if (in_dtype == DT_BF16 && out_dtype == DT_BF16)
    launch_pdl(unary_kernel<bf16, bf16>, grid, dim3(256), 0, stream, (const bf16*)in, ld_in, (bf16*)out, ld_out,
               n_rows, n_cols, kind, prm);
  else
    return NIB_ERR_BAD_ARGUMENT;
  NIB_LAUNCH_CHECK();
}
