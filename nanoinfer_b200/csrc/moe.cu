// A routed feed-forward: every row goes through `top` of `n_expert` small two-layer experts.
//   z = W_router h   (32-bit),  s = softmax(z) over all experts,  the `top` largest s are chosen
//   (ties to the lower index), their weights are those s themselves or, with `renorm`, divided by
//   their sum;  out = sum over the chosen e of s_e * W_down[e] act(W_up[e] h).
//   moe_route : a block per row -> ids [T, top], weights [T, top]
//   moe_up    : a block per (row, chosen expert, slice of the inner width): inner = act(W_up[e] h)
//   moe_down  : a block per (row, slice of the width): x += sum_j s_j W_down[e_j] inner_j   (one block owns
//               an output, so the sum has a fixed order and needs no atomics)
// Expert weights are stacked [n_expert, out, in].  A warp makes an output at a time: its lanes walk the
// input dimension, which is how the weight rows lie in memory.  Accumulation and activation are 32-bit.
//
// These three read an expert's weights again for every row that visits it, which is right for a handful of
// rows.  A step of many rows turns the loop inside out (moe_grouped): a block owns (expert, 32 outputs), keeps
// that tile of the expert's matrix in shared memory, and streams through it every row that chose the expert
// (each warp scans the step's choices for its own share of them; a lane per output, the row broadcast from
// shared memory).  The second product leaves each (row, choice)'s weighted result in a buffer of its own and
// moe_combine adds a row's choices into the stream in the order of the choices: no atomics, a fixed order.
//
// Where the experts are few for what a row chooses, a step of many rows does better still with ALL experts as two
// products of the engine's own (tensor cores): act(h . [W_up of all experts]^T) in one product, every expert's
// part of a row scaled by the row's weight for it or by 0 (moe_scale), then every expert's second matrix on its
// part, one product an expert, all adding into the stream.  n_expert / top times the arithmetic, on another
// class of unit.  (The second matrices side by side as ONE matrix [C, n_expert * F] would make that one product
// too; it was built and cost the row-by-row kernel of decode steps half its speed, its weight rows then lying
// n_expert * F apart, so the stacked layout stayed.)
//
// Variants that a model's configuration chooses: scores that are sigmoids of the logits instead of a softmax
// (`score` 1; the choice is then made on the logits themselves, which order the experts as their sigmoids do and do
// not saturate); gated experts W_down (act(W_gate h) * (W_up h)) whose first two matrices lie interleaved in one
// (row 2f the gate's, row 2f + 1 the value's: `gated`); and the chosen expert's score multiplying its INPUT instead
// of its output (the first product is linear, so the score scales its two results before the activation, and the
// second product then runs with a null `weights`).
#include <algorithm>

#include "api.h"
#include "common.cuh"

namespace nib {

constexpr int MOE_WARPS = 4;

template <typename T>
__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_route_kernel(const T* h, int ldh, const T* __restrict__ wr, int C, int n_expert, int top, int renorm, int score,
                 const float* __restrict__ choice_bias, int n_real, float* x, int* ids, float* weights) {
  pdl_trigger();
  extern __shared__ float smem[];
  float* row = smem;               // [C]
  float* prob = smem + C;          // [n_expert]
  __shared__ float scratch[32];
  __shared__ float pass_on;        // the summed scores of the chosen experts that hand their input on
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) pass_on = 0.0f;
  pdl_wait();
  for (int c = threadIdx.x; c < C; c += blockDim.x) row[c] = to_float(h[(size_t)t * ldh + c]);
  __syncthreads();
  for (int e = warp; e < n_expert; e += MOE_WARPS) {
    const T* w = wr + (size_t)e * C;
    float s = 0.0f;
    for (int c = lane; c < C; c += 32) s += row[c] * to_float(w[c]);
    s = warp_sum(s);
    if (lane == 0) prob[e] = s;
  }
  __syncthreads();
  if (score == 0) {   // softmax over all experts (score 1: the logits stay, the chosen ones' sigmoids are the scores)
    float mx = -INFINITY;
    for (int e = threadIdx.x; e < n_expert; e += blockDim.x) mx = fmaxf(mx, prob[e]);
    mx = block_max(mx, scratch);
    float sum = 0.0f;
    for (int e = threadIdx.x; e < n_expert; e += blockDim.x) sum += expf(prob[e] - mx);
    sum = block_sum(sum, scratch);
    __syncthreads();
    for (int e = threadIdx.x; e < n_expert; e += blockDim.x) prob[e] = expf(prob[e] - mx) / sum;
    __syncthreads();
  }
  if (warp == 0) {
    float total = 0.0f, handed = 0.0f;
    for (int k = 0; k < top; ++k) {
      float best = -INFINITY;
      int at = -1;
      for (int e = lane; e < n_expert; e += 32) {
        const float p = prob[e] + (choice_bias ? choice_bias[e] : 0.0f);   // (the bias moves the choice only)
        if (p > best) { best = p; at = e; }      // (a taken expert holds -inf; a NaN is never larger)
      }
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        if (oa >= 0 && (at < 0 || ob > best || (ob == best && oa < at))) { best = ob; at = oa; }
      }
      if (at < 0) { at = k % n_real; best = 0.0f; }   // rows that hold no numbers (rows of no request)
      else {
        if (choice_bias) best = prob[at];          // the weight is the score itself
        if (score == 1) best = 1.0f / (1.0f + expf(-best));
      }
      // an expert beyond the first n_real has no matrices: it hands its input on, times its score; the expert
      // kernels skip the id -1
      if (at >= n_real) handed += best;
      __syncwarp();
      if (lane == 0) {
        ids[(size_t)t * top + k] = at < n_real ? at : -1;
        weights[(size_t)t * top + k] = best;
        prob[at] = -INFINITY;
      }
      total += best;
      __syncwarp();
    }
    if (renorm && total > 0.0f) {
      for (int k = lane; k < top; k += 32) weights[(size_t)t * top + k] /= total;
      handed /= total;
    }
    if (lane == 0) pass_on = handed;
  }
  if (x != nullptr && n_real < n_expert) {
    __syncthreads();
    const float wgt = pass_on;
    if (wgt != 0.0f)
      for (int c = threadIdx.x; c < C; c += blockDim.x) x[(size_t)t * C + c] += wgt * row[c];
  }
}

constexpr int MOE_PER_WARP = 2;   // outputs a warp makes one after the other (few: a step of few rows is bound by the
                                  // latency of each weight row's loads, so it wants many warps at once)

template <typename T>
__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_up_kernel(const T* h, int ldh, const T* __restrict__ w_up, const int* ids, T* inner, int C, int F, int top,
              int act, float act_prm, int gated, const float* in_weights) {
  pdl_trigger();
  extern __shared__ float row[];   // [C]
  const int p = blockIdx.x, t = p / top, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_wait();
  const int e = ids[p];
  if (e < 0) return;               // a choice without matrices: the second product skips it too
  for (int c = threadIdx.x; c < C; c += blockDim.x) row[c] = to_float(h[(size_t)t * ldh + c]);
  __syncthreads();
  const int f0 = (blockIdx.y * MOE_WARPS + warp) * MOE_PER_WARP;
  if (gated) {   // rows 2f and 2f + 1 of the expert's matrix are output f's gate and value
    const float ws = in_weights ? in_weights[p] : 1.0f;
    for (int f = f0; f < min(F, f0 + MOE_PER_WARP); ++f) {
      const T* w = w_up + ((size_t)e * F + f) * 2 * C;
      float g = 0.0f, u = 0.0f;
      for (int c = lane; c < C; c += 32) {
        g += row[c] * to_float(w[c]);
        u += row[c] * to_float(w[C + c]);
      }
      g = warp_sum(g);
      u = warp_sum(u);
      if (lane == 0) inner[(size_t)p * F + f] = from_float<T>(gated_act(ws * g, ws * u, act, act_prm));
    }
    return;
  }
  for (int f = f0; f < min(F, f0 + MOE_PER_WARP); ++f) {
    const T* w = w_up + ((size_t)e * F + f) * C;
    float s = 0.0f;
    for (int c = lane; c < C; c += 32) s += row[c] * to_float(w[c]);
    s = warp_sum(s);
    if (lane == 0) inner[(size_t)p * F + f] = from_float<T>(apply_act(s, act));
  }
}

template <typename T>
__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_down_kernel(const T* inner, const T* __restrict__ w_down, const int* ids, const float* weights, float* x, int C,
                int F, int top) {
  pdl_trigger();
  extern __shared__ float rows[];  // [top][F]
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_wait();
  for (int i = threadIdx.x; i < top * F; i += blockDim.x)
    rows[i] = ids[(size_t)t * top + i / F] < 0 ? 0.0f : to_float(inner[(size_t)t * top * F + i]);
  __syncthreads();
  const int c0 = (blockIdx.y * MOE_WARPS + warp) * MOE_PER_WARP;
  for (int c = c0; c < min(C, c0 + MOE_PER_WARP); ++c) {
    float total = 0.0f;
    for (int k = 0; k < top; ++k) {
      const int e = ids[(size_t)t * top + k];
      if (e < 0) continue;
      const T* w = w_down + ((size_t)e * C + c) * F;
      const float* r = rows + k * F;
      float s = 0.0f;
      for (int f = lane; f < F; f += 32) s += r[f] * to_float(w[f]);
      total += (weights ? weights[(size_t)t * top + k] : 1.0f) * warp_sum(s);
    }
    if (lane == 0) x[(size_t)t * C + c] += total;
  }
}

constexpr int MOE_G_WARPS = 4, MOE_G_OUT = 32, MOE_G_ROWS = 4;

// MODE 0: out[p, n] = act(W[e][n] . src[p / top])   (src: the rows, out: T [P, N])
// MODE 1: out[p, n] = weights[p] * (W[e][n] . src[p])   (src: the inner activations [P, K], out: float [P, N]; null weights: 1)
// MODE 2: out[p, n / 2] = act(s g) * (s u), g and u the products of rows n, n + 1 (n even) of W[e] with src[p / top],
//         s = weights[p] (null: 1): gated experts, out T [P, N / 2]
// A warp collects four (row, choice) pairs of the block's expert at a time and lays their inputs side by side
// ([K][4] floats), so that one 16-byte read serves four multiply-adds beside one read of the lane's weight.
template <typename T, typename TO, int MODE>
__global__ void __launch_bounds__(MOE_G_WARPS * 32)
moe_grouped_kernel(const T* src, int ld_src, const T* __restrict__ w, const int* ids, const float* weights, TO* out,
                   int n_pairs, int top, int N, int K, int kp, int act, float act_prm, int chunk) {
  pdl_trigger();
  extern __shared__ __align__(16) unsigned char raw[];
  float4* rows = reinterpret_cast<float4*>(raw);                            // [warps][K]: four inputs side by side
  T* wt = reinterpret_cast<T*>(raw + (size_t)MOE_G_WARPS * K * sizeof(float4));   // [MOE_G_OUT][kp]: the expert's tile
  const int e = blockIdx.x, n0 = blockIdx.y * MOE_G_OUT;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* we = w + ((size_t)e * N + n0) * K;
  for (int n = warp; n < MOE_G_OUT; n += MOE_G_WARPS)
    for (int k = lane; k < K; k += 32) wt[n * kp + k] = n0 + n < N ? we[(size_t)n * K + k] : from_float<T>(0.0f);
  pdl_wait();
  __syncthreads();
  float4* row = rows + warp * K;
  const T* mine = wt + lane * kp;
  int found[MOE_G_ROWS], nf = 0;
  auto run = [&]() {                      // the products of the nf pairs in `found` with the block's tile
    const T* s[MOE_G_ROWS];
#pragma unroll
    for (int i = 0; i < MOE_G_ROWS; ++i) s[i] = src + (size_t)(i < nf ? (MODE != 1 ? found[i] / top : found[i]) : 0) * ld_src;
    __syncwarp();
#pragma unroll 4
    for (int k = lane; k < K; k += 32)
      row[k] = make_float4(to_float(s[0][k]), nf > 1 ? to_float(s[1][k]) : 0.f, nf > 2 ? to_float(s[2][k]) : 0.f,
                           nf > 3 ? to_float(s[3][k]) : 0.f);
    __syncwarp();
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int k = 0; k < K; ++k) {
      const float wv = to_float(mine[k]);
      const float4 a = row[k];
      acc.x += a.x * wv; acc.y += a.y * wv; acc.z += a.z * wv; acc.w += a.w * wv;
    }
    const float v[MOE_G_ROWS] = {acc.x, acc.y, acc.z, acc.w};
    if (MODE == 2) {   // a gate and its value lie in neighbouring lanes
#pragma unroll
      for (int i = 0; i < MOE_G_ROWS; ++i) {
        const float other = __shfl_xor_sync(0xffffffffu, v[i], 1);
        if (i < nf && !(lane & 1) && n0 + lane + 1 < N) {
          const float ws = weights ? weights[found[i]] : 1.0f;
          out[(size_t)found[i] * (N / 2) + (n0 + lane) / 2] = from_float<TO>(gated_act(ws * v[i], ws * other, act, act_prm));
        }
      }
    } else if (n0 + lane < N) {
#pragma unroll
      for (int i = 0; i < MOE_G_ROWS; ++i) {
        if (i < nf) {
          if (MODE == 0)
            out[(size_t)found[i] * N + n0 + lane] = from_float<TO>(apply_act(v[i], act));
          else
            out[(size_t)found[i] * N + n0 + lane] = from_float<TO>((weights ? weights[found[i]] : 1.0f) * v[i]);
        }
      }
    }
    nf = 0;
  };
  // a warp looks at 32 choices at a time (a lane each) and takes those of the block's expert in their order;
  // the step's choices are cut into gridDim.z chunks, a block a chunk, so that an expert that many rows chose
  // is the work of many blocks
  const int last = min(n_pairs, ((int)blockIdx.z + 1) * chunk);
  for (int base = blockIdx.z * chunk + warp * 32; base < last; base += MOE_G_WARPS * 32) {
    const int p = base + lane;
    unsigned hits = __ballot_sync(0xffffffffu, p < last && ids[p] == e);
    while (hits) {
      const int bit = __ffs(hits) - 1;
      hits &= hits - 1;
#pragma unroll
      for (int i = 0; i < MOE_G_ROWS; ++i)
        if (i == nf) found[i] = base + bit;
      if (++nf == MOE_G_ROWS) run();
    }
  }
  if (nf > 0) run();
}

// inner [T, n_expert * F]: expert e's part of row t is multiplied by the row's weight for e, by 0 where the row
// did not choose e (so that one product over all experts' second matrices adds up the chosen ones only).
template <typename T>
__global__ void __launch_bounds__(256)
moe_scale_kernel(T* inner, const int* ids, const float* weights, int n_expert, int F, int top, size_t n) {
  pdl_trigger();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const size_t t = i / ((size_t)n_expert * F);
  const int e = (int)((i / F) % n_expert);
  float s = 0.0f;
  for (int k = 0; k < top; ++k)
    if (ids[t * top + k] == e) s = weights[t * top + k];
  inner[i] = from_float<T>(s == 0.0f ? 0.0f : s * to_float(inner[i]));
}

// The gated form of the same: pre [T, n_expert * 2F] holds every expert's (gate, value) pairs side by side; inner
// [T, n_expert * F] = act(s g) * (s u) with `on_input`, else s * act(g) * u; s the row's weight for the expert, and 0
// where the row did not choose it.
template <typename TI, typename T>
__global__ void __launch_bounds__(256)
moe_gate_scale_kernel(const TI* pre, T* inner, const int* ids, const float* weights, int n_expert, int F, int top,
                      int act, float act_prm, int on_input, size_t n) {
  pdl_trigger();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const size_t t = i / ((size_t)n_expert * F);
  const int e = (int)((i / F) % n_expert);
  float s = 0.0f;
  bool chosen = false;
  for (int k = 0; k < top; ++k)
    if (ids[t * top + k] == e) { s = weights[t * top + k]; chosen = true; }
  float v = 0.0f;
  if (chosen) {
    const float g = to_float(pre[2 * i]), u = to_float(pre[2 * i + 1]);
    v = on_input ? gated_act(s * g, s * u, act, act_prm) : s * gated_act(g, u, act, act_prm);
  }
  inner[i] = from_float<T>(v);
}

__global__ void __launch_bounds__(256) moe_combine_kernel(const float* parts, const int* ids, float* x, int C, int top,
                                                          size_t n) {
  pdl_trigger();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const size_t t = i / C, c = i % C;
  float total = 0.0f;
  for (int k = 0; k < top; ++k)
    if (ids == nullptr || ids[t * top + k] >= 0) total += parts[(t * top + k) * C + c];
  x[i] += total;
}

// the padded row length of the staged tile: lanes read rows `kp` elements apart, which must fall into 32 different banks
template <typename T> static int moe_padded(int K) {
  if (sizeof(T) == 4) return K | 1;
  int kp = K + (K & 1);            // even
  return (kp / 2) % 2 ? kp : kp + 2;
}
template <typename T> static size_t moe_grouped_smem(int K) {
  return (size_t)MOE_G_OUT * moe_padded<T>(K) * sizeof(T) + (size_t)MOE_G_WARPS * K * sizeof(float4);
}

template <typename T, typename TO, int MODE>
static int launch_moe_grouped(const T* src, int ld_src, const T* w, const int* ids, const float* weights, TO* out,
                              int n_pairs, int top, int n_expert, int N, int K, int act, float act_prm, cudaStream_t stream) {
  const size_t smem = moe_grouped_smem<T>(K);
  if (smem > 200 * 1024) return NIB_ERR_UNSUPPORTED_SIZE;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(moe_grouped_kernel<T, TO, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  // chunks of the choices: about 32 choices of the block's expert a block if the choices were even
  const int z = std::max(1, std::min(64, n_pairs / (32 * n_expert)));
  const int chunk = ((n_pairs + z - 1) / z + 31) / 32 * 32;
  launch_pdl(moe_grouped_kernel<T, TO, MODE>, dim3(n_expert, (N + MOE_G_OUT - 1) / MOE_G_OUT, (n_pairs + chunk - 1) / chunk),
             dim3(MOE_G_WARPS * 32), smem, stream, src, ld_src, w, ids, weights, out, n_pairs, top, N, K,
             moe_padded<T>(K), act, act_prm, chunk);
  NIB_LAUNCH_CHECK();
}

}  // namespace nib

using namespace nib;

// The expert-major form of nib_moe_up (phase 0; phase 3: gated, N = 2F interleaved rows, out [T * top, F], `weights`
// scaling the inputs), nib_moe_down into `parts` float [T * top, C] (phase 1), and the sum of
// a row's parts into the stream (phase 2).  -2 where a tile of an expert's matrix does not fit shared memory.
extern "C" int nib_moe_grouped(int dtype, int phase, const void* src, int ld_src, const void* w, const int* ids,
                               const float* weights, void* out, float* x, int T, int top, int n_expert, int N, int K,
                               int act, float act_prm, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (phase == 2) {
    const size_t n = (size_t)T * N;
    launch_pdl(moe_combine_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, (const float*)src, ids, x, N, top, n);
    NIB_LAUNCH_CHECK();
  }
  if (dtype == DT_F32) {
    if (phase == 3)
      return launch_moe_grouped<float, float, 2>((const float*)src, ld_src, (const float*)w, ids, weights, (float*)out,
                                                 T * top, top, n_expert, N, K, act, act_prm, stream);
    if (phase == 0)
      return launch_moe_grouped<float, float, 0>((const float*)src, ld_src, (const float*)w, ids, weights, (float*)out,
                                                 T * top, top, n_expert, N, K, act, act_prm, stream);
    return launch_moe_grouped<float, float, 1>((const float*)src, ld_src, (const float*)w, ids, weights, (float*)out,
                                               T * top, top, n_expert, N, K, act, act_prm, stream);
  }
  if (dtype == DT_BF16) {
    if (phase == 3)
      return launch_moe_grouped<bf16, bf16, 2>((const bf16*)src, ld_src, (const bf16*)w, ids, weights, (bf16*)out,
                                               T * top, top, n_expert, N, K, act, act_prm, stream);
    if (phase == 0)
      return launch_moe_grouped<bf16, bf16, 0>((const bf16*)src, ld_src, (const bf16*)w, ids, weights, (bf16*)out,
                                               T * top, top, n_expert, N, K, act, act_prm, stream);
    return launch_moe_grouped<bf16, float, 1>((const bf16*)src, ld_src, (const bf16*)w, ids, weights, (float*)out,
                                              T * top, top, n_expert, N, K, act, act_prm, stream);
  }
  return NIB_ERR_BAD_ARGUMENT;
}

extern "C" int nib_moe_route(int dtype, const void* h, int ldh, const void* w_router, int T, int C, int n_expert,
                             int top, int renorm, int score, const float* choice_bias, int n_real, float* x, int* ids,
                             float* weights, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (top <= 0 || top > n_expert || C <= 0 || (score != 0 && score != 1)) return NIB_ERR_BAD_ARGUMENT;
  if (n_real <= 0 || n_real > n_expert || (n_real < n_expert && x == nullptr)) return NIB_ERR_BAD_ARGUMENT;
  const size_t smem = (size_t)(C + n_expert) * sizeof(float);
  if (smem > 200 * 1024) return NIB_ERR_UNSUPPORTED_SIZE;
  if (dtype == DT_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_route_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(moe_route_kernel<float>, dim3(T), dim3(MOE_WARPS * 32), smem, stream, (const float*)h, ldh,
               (const float*)w_router, C, n_expert, top, renorm, score, choice_bias, n_real, x, ids, weights);
  } else if (dtype == DT_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_route_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(moe_route_kernel<bf16>, dim3(T), dim3(MOE_WARPS * 32), smem, stream, (const bf16*)h, ldh,
               (const bf16*)w_router, C, n_expert, top, renorm, score, choice_bias, n_real, x, ids, weights);
  } else {
    return NIB_ERR_BAD_ARGUMENT;
  }
  NIB_LAUNCH_CHECK();
}

// inner: [T * top, F] in `dtype`; act: an activation code.  gated: w_up is [experts, 2F, C] with rows 2f, 2f + 1 the
// gate and value of output f, and in_weights (may be null) [T * top] scale the inputs.
extern "C" int nib_moe_up(int dtype, const void* h, int ldh, const void* w_up, const int* ids, void* inner, int T,
                          int C, int F, int top, int act, float act_prm, int gated, const float* in_weights, cudaStream_t stream) {
  if (T <= 0) return 0;
  const size_t smem = (size_t)C * sizeof(float);
  if (smem > 200 * 1024) return NIB_ERR_UNSUPPORTED_SIZE;
  const dim3 grid(T * top, (F + MOE_WARPS * MOE_PER_WARP - 1) / (MOE_WARPS * MOE_PER_WARP));
  if (grid.y > 65535) return NIB_ERR_UNSUPPORTED_SIZE;
  if (dtype == DT_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_up_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(moe_up_kernel<float>, grid, dim3(MOE_WARPS * 32), smem, stream, (const float*)h, ldh,
               (const float*)w_up, ids, (float*)inner, C, F, top, act, act_prm, gated, in_weights);
  } else if (dtype == DT_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_up_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(moe_up_kernel<bf16>, grid, dim3(MOE_WARPS * 32), smem, stream, (const bf16*)h, ldh, (const bf16*)w_up,
               ids, (bf16*)inner, C, F, top, act, act_prm, gated, in_weights);
  } else {
    return NIB_ERR_BAD_ARGUMENT;
  }
  NIB_LAUNCH_CHECK();
}

// x: the 32-bit residual stream [T, C]; the experts' weighted outputs are added to it.
extern "C" int nib_moe_down(int dtype, const void* inner, const void* w_down, const int* ids, const float* weights,
                            float* x, int T, int C, int F, int top, cudaStream_t stream) {
  if (T <= 0) return 0;
  const size_t smem = (size_t)top * F * sizeof(float);
  if (smem > 200 * 1024) return NIB_ERR_UNSUPPORTED_SIZE;
  const dim3 grid(T, (C + MOE_WARPS * MOE_PER_WARP - 1) / (MOE_WARPS * MOE_PER_WARP));
  if (grid.y > 65535) return NIB_ERR_UNSUPPORTED_SIZE;
  if (dtype == DT_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_down_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(moe_down_kernel<float>, grid, dim3(MOE_WARPS * 32), smem, stream, (const float*)inner,
               (const float*)w_down, ids, weights, x, C, F, top);
  } else if (dtype == DT_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_down_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(moe_down_kernel<bf16>, grid, dim3(MOE_WARPS * 32), smem, stream, (const bf16*)inner,
               (const bf16*)w_down, ids, weights, x, C, F, top);
  } else {
    return NIB_ERR_BAD_ARGUMENT;
  }
  NIB_LAUNCH_CHECK();
}

// pre: [T, n_expert * 2F] in `pre_dtype` (32-bit floats or `dtype`); inner [T, n_expert * F] in `dtype`.
extern "C" int nib_moe_gate_scale(int pre_dtype, int dtype, const void* pre, void* inner, const int* ids,
                                  const float* weights, int T, int n_expert, int F, int top, int act, float act_prm,
                                  int on_input, cudaStream_t stream) {
  if (T <= 0) return 0;
  const size_t n = (size_t)T * n_expert * F;
  const dim3 grid((unsigned)((n + 255) / 256));
  if (pre_dtype == DT_F32 && dtype == DT_F32)
    launch_pdl(moe_gate_scale_kernel<float, float>, grid, dim3(256), 0, stream, (const float*)pre, (float*)inner, ids,
               weights, n_expert, F, top, act, act_prm, on_input, n);
  else if (pre_dtype == DT_F32 && dtype == DT_BF16)
    launch_pdl(moe_gate_scale_kernel<float, bf16>, grid, dim3(256), 0, stream, (const float*)pre, (bf16*)inner, ids,
               weights, n_expert, F, top, act, act_prm, on_input, n);
  else if (pre_dtype == DT_BF16 && dtype == DT_BF16)
    launch_pdl(moe_gate_scale_kernel<bf16, bf16>, grid, dim3(256), 0, stream, (const bf16*)pre, (bf16*)inner, ids,
               weights, n_expert, F, top, act, act_prm, on_input, n);
  else
    return NIB_ERR_BAD_ARGUMENT;
  NIB_LAUNCH_CHECK();
}

extern "C" int nib_moe_scale(int dtype, void* inner, const int* ids, const float* weights, int T, int n_expert, int F,
                             int top, cudaStream_t stream) {
  if (T <= 0) return 0;
  const size_t n = (size_t)T * n_expert * F;
  const dim3 grid((unsigned)((n + 255) / 256));
  if (dtype == DT_F32)
    launch_pdl(moe_scale_kernel<float>, grid, dim3(256), 0, stream, (float*)inner, ids, weights, n_expert, F, top, n);
  else if (dtype == DT_BF16)
    launch_pdl(moe_scale_kernel<bf16>, grid, dim3(256), 0, stream, (bf16*)inner, ids, weights, n_expert, F, top, n);
  else
    return NIB_ERR_BAD_ARGUMENT;
  NIB_LAUNCH_CHECK();
}
