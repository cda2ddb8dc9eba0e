// Recurrent mixers with a matrix state per head and one decay per head and token: the gated delta rule and the
// state-space recurrence of Mamba-2, with the short causal convolution that both put ahead of it and the gated
// norm that both put behind it.
//
// Per head, with S an N x V matrix (N key channels, V value channels), a decay a_t in (0, 1] and a strength w_t:
//   gated delta rule:   S <- a S;   u = w (v - S^T k);   S <- S + k u^T;   o = S^T q       (w = beta)
//   state space:        S <- a S + k (w v)^T;   o = S^T q + D v                           (k = B, q = C, w = dt)
// The columns of S do not see one another, so a column is owned by four neighbouring threads (N / 4 values each in
// registers; the two sums over N are two shuffles each) and a block of 128 threads owns 32 columns of one head of
// one batch entry, walking the entry's rows in order.  The rows' vectors come through a double buffer in shared
// memory, eight rows at a time by cp.async.  State, decays, strengths and every sum are 32-bit.
//
// State per request (one row of the slot tensor): [taps - 1][channels] inputs of the convolution, oldest first,
// then [head][V][NP] with NP = N rounded up to what the kernel variant holds (a multiple of 16).
#include "api.h"
#include "common.cuh"

namespace nib {

__device__ __forceinline__ float softplus_f32(float v) { return v > 20.0f ? v : log1pf(expf(v)); }
__device__ __forceinline__ float silu_f32(float v) { return v / (1.0f + expf(-v)); }

// ------------------------------------------------------------------ short causal convolution over time
// out[t, c] = act(bias[c] + sum_j w[c, j] x[t - (taps - 1 - j), c]) for the channels c_off .. c_off + Cn - 1 of proj;
// inputs before the entry's first row come from the request's state (zeros at the start of a sequence).
// SHIFT: every entry of the step has one row, and the thread also moves the state on by that row.
// out16 (may be null): the same values once more as bfloat16, for a matrix product that reads them.
template <bool SHIFT>
__global__ void __launch_bounds__(256)
short_conv_kernel(const float* proj, int ld, int c_off, int Cn, int taps, const float* __restrict__ w,
                  const float* __restrict__ bias, float* state, long long state_stride,
                  const int* __restrict__ row_entry, const int* __restrict__ entry_start,
                  const int* __restrict__ entry_slot, float* out, int ldo, int act, bf16* out16, int ld16) {
  pdl_trigger();
  const int t = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  const int e = row_entry[t];
  if (e < 0 || c >= Cn) return;
  const int i = t - entry_start[e];
  float* st = state + (size_t)entry_slot[e] * state_stride;
  float acc = bias ? bias[c] : 0.0f;
  pdl_wait();
  for (int j = 0; j < taps; ++j) {
    const int src = i - (taps - 1 - j);
    const float xv = src >= 0 ? proj[(size_t)(t - (taps - 1 - j)) * ld + c_off + c] : st[(size_t)(taps - 1 + src) * Cn + c];
    acc = fmaf(w[(size_t)c * taps + j], xv, acc);
  }
  const float y = act == ACT_SILU ? silu_f32(acc) : acc;
  out[(size_t)t * ldo + c] = y;
  if (out16 != nullptr) out16[(size_t)t * ld16 + c] = __float2bfloat16_rn(y);   // for a product that follows
  if (SHIFT) {
    for (int s = 0; s + 2 < taps; ++s) st[(size_t)s * Cn + c] = st[(size_t)(s + 1) * Cn + c];
    if (taps > 1) st[(size_t)(taps - 2) * Cn + c] = proj[(size_t)t * ld + c_off + c];
  }
}

// The state after a step: the last taps - 1 inputs of [old state ; the entry's rows].  A thread owns a channel of an
// entry and writes slot s after it has read everything at or behind s + 1.
__global__ void __launch_bounds__(256)
short_conv_state_kernel(const float* proj, int ld, int c_off, int Cn, int taps, float* state, long long state_stride,
                        const int* __restrict__ entry_start, const int* __restrict__ entry_slot) {
  pdl_trigger();
  const int e = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= Cn) return;
  const int r0 = entry_start[e], n = entry_start[e + 1] - r0;
  float* st = state + (size_t)entry_slot[e] * state_stride;
  pdl_wait();
  for (int s = 0; s + 1 < taps; ++s) {
    const int idx = n + s;   // place in [old state ; rows]
    st[(size_t)s * Cn + c] = idx < taps - 1 ? st[(size_t)idx * Cn + c]
                                            : proj[(size_t)(r0 + idx - (taps - 1)) * ld + c_off + c];
  }
}

// ------------------------------------------------------------------ what the recurrence reads besides its vectors
// A warp per (row, unit).  Units 0 .. n_head - 1: the head's decay and strength,
//   delta:  a = exp(-exp(A_log) softplus(raw_a + dt_bias)),  w = sigmoid(raw_w);
//   space:  w = softplus(raw_w + dt_bias),                   a = exp(-exp(A_log) w);
// (raw_a, raw_w: columns a_off + h, w_off + h of proj).  Delta only, units n_head ..: a query or key head of the
// convolution's output is made a unit vector, x / sqrt(sum x^2 + 1e-6), queries also times N^-1/2, in place.
__global__ void __launch_bounds__(128)
scan_prepare_kernel(const float* proj, int ld, int a_off, int w_off, const float* __restrict__ A_log,
                    const float* __restrict__ dt_bias, float* cv, int ldc, int q_off, int k_off, int N, int n_head,
                    int n_kq, int delta, float* coef, int T) {
  pdl_trigger();
  const int t = blockIdx.y, lane = threadIdx.x & 31;
  const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int n_units = n_head + (delta ? 2 * n_kq : 0);
  if (unit >= n_units) return;
  pdl_wait();
  if (unit < n_head) {
    if (lane == 0) {
      const int h = unit;
      const float* p = proj + (size_t)t * ld;
      float a, wgt;
      if (delta) {
        a = expf(-expf(A_log[h]) * softplus_f32(p[a_off + h] + dt_bias[h]));
        wgt = 1.0f / (1.0f + expf(-p[w_off + h]));
      } else {
        wgt = softplus_f32(p[w_off + h] + dt_bias[h]);
        a = expf(-expf(A_log[h]) * wgt);
      }
      coef[((size_t)t * n_head + h) * 2] = a;
      coef[((size_t)t * n_head + h) * 2 + 1] = wgt;
    }
    return;
  }
  const int u = unit - n_head;
  const bool is_q = u < n_kq;
  float* x = cv + (size_t)t * ldc + (is_q ? q_off + u * N : k_off + (u - n_kq) * N);
  float ss = 0.0f;
  for (int d = lane; d < N; d += 32) ss += x[d] * x[d];
  float r = 1.0f / sqrtf(warp_sum(ss) + 1e-6f);
  if (is_q) r *= 1.0f / sqrtf((float)N);
  for (int d = lane; d < N; d += 32) x[d] *= r;
}

// ------------------------------------------------------------------ the recurrence
constexpr int SCAN_ROWS = 8;      // rows staged at a time
constexpr int SCAN_COLS = 32;     // columns of S a block owns

__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gmem_src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(gmem_src) : "memory");
}

// cv [T, ldc]: the rows' vectors: q (or C) of key/query head g at q_off + g N, k (or B) at k_off + g N, v (or x) of
// head h at v_off + h V; head h reads key/query head h / kq_ratio.  coef [T, n_head, 2]: (a, w).  out [T, ldo]
// float: o of head h at h V.  NPT: values of a column per thread (N <= 4 NPT).
template <int NPT, bool DELTA>
__global__ void __launch_bounds__(128)
gated_scan_kernel(const float* cv, int ldc, int q_off, int k_off, int v_off, int N, int V, int n_head, int kq_ratio,
                  const float* coef, const float* __restrict__ skip, float* state, long long state_stride,
                  long long s_off, const int* __restrict__ entry_start, const int* __restrict__ entry_slot,
                  float* out, int ldo, int vec4) {
  constexpr int NP = 4 * NPT;
  constexpr int ROW_F = 2 * NP + SCAN_COLS + 4;   // k | q | v | a, w, -, -
  pdl_trigger();
  extern __shared__ __align__(16) float sm[];
  const int e = blockIdx.z, h = blockIdx.y, col0 = blockIdx.x * SCAN_COLS;
  const int tid = threadIdx.x, p = tid & 3, jl = tid >> 2;
  const int j = col0 + jl;
  const bool has_col = j < V;
  const int r0 = entry_start[e], n = entry_start[e + 1] - r0;
  const int g = h / kq_ratio;
  const int n_cols = min(SCAN_COLS, V - col0);
  for (int i = tid; i < 2 * SCAN_ROWS * ROW_F; i += 128) sm[i] = 0.0f;   // (the tails behind N and V stay zero)
  // the state belongs to this kernel alone: what it holds was written a step ago
  float S[NPT];
  float* sp = state + (size_t)entry_slot[e] * state_stride + s_off + ((size_t)h * V + (has_col ? j : 0)) * NP;
#pragma unroll
  for (int i = 0; i < NPT / 4; ++i) {
    const float4 s4 = has_col ? *reinterpret_cast<const float4*>(sp + 16 * i + 4 * p) : make_float4(0.f, 0.f, 0.f, 0.f);
    S[4 * i] = s4.x; S[4 * i + 1] = s4.y; S[4 * i + 2] = s4.z; S[4 * i + 3] = s4.w;
  }
  const float d_skip = (!DELTA && skip != nullptr) ? skip[h] : 0.0f;
  __syncthreads();
  pdl_wait();

  // asks for the rows of chunk ck into buffer b
  auto stage = [&](int ck, int b) {
    float* base = sm + (size_t)b * SCAN_ROWS * ROW_F;
    const int rows = min(SCAN_ROWS, n - ck * SCAN_ROWS);
    if (vec4) {
      const int nk = N >> 2, nv = n_cols >> 2, per = 2 * nk + nv;
      for (int i = tid; i < rows * per; i += 128) {
        const int rr = i / per, x = i % per;
        const float* src = cv + (size_t)(r0 + ck * SCAN_ROWS + rr) * ldc;
        float* dst = base + rr * ROW_F;
        if (x < nk) cp_async16(dst + 4 * x, src + k_off + g * N + 4 * x, true);
        else if (x < 2 * nk) cp_async16(dst + NP + 4 * (x - nk), src + q_off + g * N + 4 * (x - nk), true);
        else cp_async16(dst + 2 * NP + 4 * (x - 2 * nk), src + v_off + h * V + col0 + 4 * (x - 2 * nk), true);
      }
    } else {
      const int per = 2 * N + n_cols;
      for (int i = tid; i < rows * per; i += 128) {
        const int rr = i / per, x = i % per;
        const float* src = cv + (size_t)(r0 + ck * SCAN_ROWS + rr) * ldc;
        float* dst = base + rr * ROW_F;
        if (x < N) cp_async4(dst + x, src + k_off + g * N + x);
        else if (x < 2 * N) cp_async4(dst + NP + (x - N), src + q_off + g * N + (x - N));
        else cp_async4(dst + 2 * NP + (x - 2 * N), src + v_off + h * V + col0 + (x - 2 * N));
      }
    }
    for (int i = tid; i < rows * 2; i += 128)
      cp_async4(base + (i >> 1) * ROW_F + 2 * NP + SCAN_COLS + (i & 1),
                coef + ((size_t)(r0 + ck * SCAN_ROWS + (i >> 1)) * n_head + h) * 2 + (i & 1));
    cp_async_commit();
  };

  const int n_chunks = (n + SCAN_ROWS - 1) / SCAN_ROWS;
  if (n_chunks > 0) stage(0, 0);
  for (int ck = 0; ck < n_chunks; ++ck) {
    cp_async_wait<0>();
    __syncthreads();   // chunk ck has arrived, and every thread is done with the buffer that chunk ck + 1 goes to
    if (ck + 1 < n_chunks) stage(ck + 1, (ck + 1) & 1);
    const float* base = sm + (size_t)(ck & 1) * SCAN_ROWS * ROW_F;
    const int rows = min(SCAN_ROWS, n - ck * SCAN_ROWS);
    float o[SCAN_ROWS], vj[SCAN_ROWS];
#pragma unroll
    for (int rr = 0; rr < SCAN_ROWS; ++rr) {
      o[rr] = 0.0f;
      vj[rr] = 0.0f;
      if (rr < rows) {
        const float* kr = base + rr * ROW_F;
        const float* qr = kr + NP;
        const float a = kr[2 * NP + SCAN_COLS], wgt = kr[2 * NP + SCAN_COLS + 1];
        vj[rr] = kr[2 * NP + jl];
        float u;
        if (DELTA) {
          float ks = 0.0f;
#pragma unroll
          for (int i = 0; i < NPT / 4; ++i) {
            const float4 k4 = *reinterpret_cast<const float4*>(kr + 16 * i + 4 * p);
            ks = fmaf(k4.x, S[4 * i], ks); ks = fmaf(k4.y, S[4 * i + 1], ks);
            ks = fmaf(k4.z, S[4 * i + 2], ks); ks = fmaf(k4.w, S[4 * i + 3], ks);
          }
          ks += __shfl_xor_sync(0xffffffffu, ks, 1);
          ks += __shfl_xor_sync(0xffffffffu, ks, 2);
          u = wgt * (vj[rr] - a * ks);
        } else {
          u = wgt * vj[rr];
        }
        float acc = 0.0f;
#pragma unroll
        for (int i = 0; i < NPT / 4; ++i) {
          const float4 k4 = *reinterpret_cast<const float4*>(kr + 16 * i + 4 * p);
          const float4 q4 = *reinterpret_cast<const float4*>(qr + 16 * i + 4 * p);
          S[4 * i] = fmaf(a, S[4 * i], k4.x * u);         acc = fmaf(q4.x, S[4 * i], acc);
          S[4 * i + 1] = fmaf(a, S[4 * i + 1], k4.y * u); acc = fmaf(q4.y, S[4 * i + 1], acc);
          S[4 * i + 2] = fmaf(a, S[4 * i + 2], k4.z * u); acc = fmaf(q4.z, S[4 * i + 2], acc);
          S[4 * i + 3] = fmaf(a, S[4 * i + 3], k4.w * u); acc = fmaf(q4.w, S[4 * i + 3], acc);
        }
        o[rr] = acc;
      }
    }
    // the read-outs' sums over the four threads of a column, off the chain from row to row
#pragma unroll
    for (int rr = 0; rr < SCAN_ROWS; ++rr) {
      o[rr] += __shfl_xor_sync(0xffffffffu, o[rr], 1);
      o[rr] += __shfl_xor_sync(0xffffffffu, o[rr], 2);
      if (rr < rows && p == 0 && has_col)
        out[(size_t)(r0 + ck * SCAN_ROWS + rr) * ldo + h * V + j] = o[rr] + d_skip * vj[rr];
    }
  }
  if (has_col) {
#pragma unroll
    for (int i = 0; i < NPT / 4; ++i)
      *reinterpret_cast<float4*>(sp + 16 * i + 4 * p) = make_float4(S[4 * i], S[4 * i + 1], S[4 * i + 2], S[4 * i + 3]);
  }
}

// ------------------------------------------------------------------ the gated norm behind the recurrence
// A block per (row, group of gs values): y = o (times silu(gate) first where gate_first), y / sqrt(mean(y^2) + eps)
// times weight[(index in the row) mod wlen] (times silu(gate) afterwards where !gate_first), times out_scale.
template <typename OutT>
__global__ void __launch_bounds__(128)
gated_norm_kernel(const float* o, int ldo, const float* gate, int ldg, const float* __restrict__ weight, int wlen,
                  int gs, float eps, int gate_first, float out_scale, OutT* out, int ld_out) {
  pdl_trigger();
  __shared__ float scratch[32];
  const int t = blockIdx.y, c0 = blockIdx.x * gs;
  pdl_wait();
  const float* orow = o + (size_t)t * ldo + c0;
  const float* grow = gate ? gate + (size_t)t * ldg + c0 : nullptr;
  float ss = 0.0f;
  for (int c = threadIdx.x; c < gs; c += blockDim.x) {
    float y = orow[c];
    if (gate_first && grow) y *= silu_f32(grow[c]);
    ss += y * y;
  }
  const float r = 1.0f / sqrtf(block_sum(ss, scratch) / (float)gs + eps);
  for (int c = threadIdx.x; c < gs; c += blockDim.x) {
    float y = orow[c];
    if (gate_first && grow) y *= silu_f32(grow[c]);
    y = y * r * weight[(c0 + c) % wlen];
    if (!gate_first && grow) y *= silu_f32(grow[c]);
    out[(size_t)t * ld_out + c0 + c] = from_float<OutT>(y * out_scale);
  }
}

}  // namespace nib

using namespace nib;

// fused != 0: every entry of the step is one row (T == n_entries): the convolution also moves the state on.
extern "C" int nib_short_conv(const float* proj, int ld, int c_off, int Cn, int taps, const float* w, const float* bias,
                              float* state, long long state_stride, const int* row_entry, const int* entry_start,
                              const int* entry_slot, float* out, int ldo, int T, int n_entries, int act, int fused,
                              void* out16, int ld16, cudaStream_t stream) {
  if (T <= 0 || Cn <= 0) return 0;
  if (taps < 1 || taps > 64 || T > 65535 || n_entries > 65535) return NIB_ERR_UNSUPPORTED_SIZE;
  const dim3 grid((Cn + 255) / 256, T);
  if (fused) {
    launch_pdl(short_conv_kernel<true>, grid, dim3(256), 0, stream, proj, ld, c_off, Cn, taps, w, bias, state,
               state_stride, row_entry, entry_start, entry_slot, out, ldo, act, (bf16*)out16, ld16);
    NIB_LAUNCH_CHECK();
  }
  launch_pdl(short_conv_kernel<false>, grid, dim3(256), 0, stream, proj, ld, c_off, Cn, taps, w, bias, state,
             state_stride, row_entry, entry_start, entry_slot, out, ldo, act, (bf16*)out16, ld16);
  if (taps > 1 && n_entries > 0)
    launch_pdl(short_conv_state_kernel, dim3((Cn + 255) / 256, n_entries), dim3(256), 0, stream, proj, ld, c_off, Cn,
               taps, state, state_stride, entry_start, entry_slot);
  NIB_LAUNCH_CHECK();
}

extern "C" int nib_scan_prepare(const float* proj, int ld, int a_off, int w_off, const float* A_log,
                                const float* dt_bias, float* cv, int ldc, int q_off, int k_off, int N, int n_head,
                                int n_kq, int delta, float* coef, int T, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (T > 65535) return NIB_ERR_UNSUPPORTED_SIZE;
  const int units = n_head + (delta ? 2 * n_kq : 0);
  launch_pdl(scan_prepare_kernel, dim3((units + 3) / 4, T), dim3(128), 0, stream, proj, ld, a_off, w_off, A_log,
             dt_bias, cv, ldc, q_off, k_off, N, n_head, n_kq, delta, coef, T);
  NIB_LAUNCH_CHECK();
}

// N rounded up to what a kernel variant holds (0: too large)
extern "C" int nib_gated_scan_padded(int N) {
  const int sizes[] = {16, 32, 48, 64, 96, 128, 192, 256};
  for (int s : sizes)
    if (N <= s) return s;
  return 0;
}

template <int NPT>
static int launch_scan(int delta, dim3 grid, cudaStream_t stream, const float* cv, int ldc, int q_off, int k_off,
                       int v_off, int N, int V, int n_head, int kq_ratio, const float* coef, const float* skip,
                       float* state, long long state_stride, long long s_off, const int* entry_start,
                       const int* entry_slot, float* out, int ldo, int vec4) {
  const size_t smem = (size_t)2 * SCAN_ROWS * (2 * 4 * NPT + SCAN_COLS + 4) * sizeof(float);
  if (delta) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(gated_scan_kernel<NPT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(gated_scan_kernel<NPT, true>, grid, dim3(128), smem, stream, cv, ldc, q_off, k_off, v_off, N, V, n_head,
               kq_ratio, coef, skip, state, state_stride, s_off, entry_start, entry_slot, out, ldo, vec4);
  } else {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(gated_scan_kernel<NPT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(gated_scan_kernel<NPT, false>, grid, dim3(128), smem, stream, cv, ldc, q_off, k_off, v_off, N, V, n_head,
               kq_ratio, coef, skip, state, state_stride, s_off, entry_start, entry_slot, out, ldo, vec4);
  }
  NIB_LAUNCH_CHECK();
}

// s_off: floats from the start of a slot's row to the matrices [n_head][V][nib_gated_scan_padded(N)].
extern "C" int nib_gated_scan(int delta, const float* cv, int ldc, int q_off, int k_off, int v_off, int N, int V,
                              int n_head, int kq_ratio, const float* coef, const float* skip, float* state,
                              long long state_stride, long long s_off, const int* entry_start, const int* entry_slot,
                              int n_entries, float* out, int ldo, cudaStream_t stream) {
  if (n_entries <= 0) return 0;
  const int NP = nib_gated_scan_padded(N);
  if (NP == 0 || N <= 0 || V <= 0 || n_head > 65535 || n_entries > 65535) return NIB_ERR_UNSUPPORTED_SIZE;
  if (kq_ratio <= 0 || n_head % kq_ratio != 0 || (s_off & 3) || (state_stride & 3)) return NIB_ERR_BAD_ARGUMENT;
  const int vec4 = !((N | V | ldc | q_off | k_off | v_off) & 3) && (((uintptr_t)cv & 15) == 0);
  const dim3 grid((V + SCAN_COLS - 1) / SCAN_COLS, n_head, n_entries);
#define NIB_SCAN(NPT) return launch_scan<NPT>(delta, grid, stream, cv, ldc, q_off, k_off, v_off, N, V, n_head, kq_ratio, \
                                              coef, skip, state, state_stride, s_off, entry_start, entry_slot, out, ldo, vec4)
  switch (NP) {
    case 16: NIB_SCAN(4);
    case 32: NIB_SCAN(8);
    case 48: NIB_SCAN(12);
    case 64: NIB_SCAN(16);
    case 96: NIB_SCAN(24);
    case 128: NIB_SCAN(32);
    case 192: NIB_SCAN(48);
    default: NIB_SCAN(64);
  }
#undef NIB_SCAN
}

extern "C" int nib_gated_norm(int out_dtype, const float* o, int ldo, const float* gate, int ldg, const float* weight,
                              int wlen, int n_groups, int gs, float eps, int gate_first, float out_scale, void* out,
                              int ld_out, int T, cudaStream_t stream) {
  if (T <= 0 || n_groups <= 0) return 0;
  if (gs <= 0 || wlen <= 0 || T > 65535) return NIB_ERR_UNSUPPORTED_SIZE;
  const dim3 grid(n_groups, T);
  if (out_dtype == DT_F32)
    launch_pdl(gated_norm_kernel<float>, grid, dim3(128), 0, stream, o, ldo, gate, ldg, weight, wlen, gs, eps, gate_first,
               out_scale, (float*)out, ld_out);
  else if (out_dtype == DT_BF16)
    launch_pdl(gated_norm_kernel<bf16>, grid, dim3(128), 0, stream, o, ldo, gate, ldg, weight, wlen, gs, eps, gate_first,
               out_scale, (bf16*)out, ld_out);
  else
    return NIB_ERR_BAD_ARGUMENT;
  NIB_LAUNCH_CHECK();
}
