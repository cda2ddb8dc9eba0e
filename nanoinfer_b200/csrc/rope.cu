// Rotary positions on queries and keys, fused with what follows the q/k/v projection of an attention layer:
// the cast to the engine's dtype, the padding of a head to the cache's head size, and the append of keys and
// values to their slots of the paged cache.
//
// A head's first `rot_dims` values turn in pairs (2i, 2i + 1) (the interleaved layout) by the angle
// a = position * freqs[i]:   (u, w) -> (u cos a - w sin a, w cos a + u sin a);   the other values pass.
// The angle and its sine and cosine are made in double precision from a table of frequencies that the host
// computed in double precision, so that a position of many thousands loses nothing.
//
// proj [T, ld] float: a row holds [q: n_head x dim | k: n_kv_head x dim | v: n_kv_head x vdim] at q_off, k_off,
// v_off.  q_out [T, ldq] receives n_head heads of `hd` values (dim values, then zeros); the cache layer
// [n_pages, 2, n_kv_head, page_size, hd] receives the row's keys (plane 0) and values (plane 1), padded
// likewise.  Rows of no request (row_entry < 0) write their queries only.  A block a row; a thread owns pair i of
// every n-th head.
#include "api.h"
#include "common.cuh"

namespace nib {

template <typename T>
__device__ __forceinline__ void store_pair(T* p, float a, float b);
template <>
__device__ __forceinline__ void store_pair<float>(float* p, float a, float b) {
  *reinterpret_cast<float2*>(p) = make_float2(a, b);
}
template <>
__device__ __forceinline__ void store_pair<bf16>(bf16* p, float a, float b) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

template <typename T>
__global__ void __launch_bounds__(256)
rope_append_kernel(const float* proj, int ld, int q_off, int k_off, int v_off, int n_head, int n_kv_head, int dim,
                   int vdim, int hd, int rot_dims, const double* __restrict__ freqs, const int* __restrict__ positions,
                   const int* __restrict__ row_entry, T* q_out, int ldq, T* cache, const int* __restrict__ block_table,
                   int max_blocks, int page_size, int n_pages, int* status) {
  pdl_trigger();
  const int t = blockIdx.x;
  const int pos = positions[t], entry = row_entry[t];
  T* k_dst = nullptr;
  T* v_dst = nullptr;
  if (entry >= 0 && cache != nullptr) {
    const int page = block_table[(size_t)entry * max_blocks + pos / page_size];
    if (page < 0 || page >= n_pages) {
      if (threadIdx.x == 0) *status = NIB_STATUS_BAD_PAGE;
    } else {
      k_dst = cache + kv_offset(page, 0, 0, pos % page_size, n_kv_head, page_size, hd);
      v_dst = cache + kv_offset(page, 1, 0, pos % page_size, n_kv_head, page_size, hd);
    }
  }
  const size_t head_stride = (size_t)page_size * hd;   // from one key/value head's row to the next head's
  pdl_wait();
  const float* p = proj + (size_t)t * ld;
  // a thread owns pair i of every n-th head (queries, then keys, then values), n = groups of hd / 2 threads a block
  const int half = hd / 2, i = threadIdx.x % half, group = threadIdx.x / half, n_groups = blockDim.x / half;
  if (group >= n_groups) return;
  float c = 1.0f, s = 0.0f;
  if (2 * i < rot_dims) {
    double sd, cd;
    sincos((double)pos * freqs[i], &sd, &cd);
    c = (float)cd;
    s = (float)sd;
  }
  const bool in_k = 2 * i < dim, in_v = 2 * i < vdim;
  for (int hh = group; hh < n_head + 2 * n_kv_head; hh += n_groups) {
    if (hh < n_head + n_kv_head) {             // a query or a key head: rotated
      const bool is_q = hh < n_head;
      const int h = is_q ? hh : hh - n_head;
      if (!is_q && k_dst == nullptr) continue;
      float u = 0.0f, w = 0.0f;
      if (in_k) {
        const float2 x = *reinterpret_cast<const float2*>(p + (is_q ? q_off : k_off) + h * dim + 2 * i);
        u = x.x * c - x.y * s;
        w = x.y * c + x.x * s;
      }
      store_pair<T>(is_q ? q_out + (size_t)t * ldq + h * hd + 2 * i : k_dst + h * head_stride + 2 * i, u, w);
    } else if (v_dst != nullptr) {
      const int h = hh - n_head - n_kv_head;
      float2 y = make_float2(0.0f, 0.0f);
      if (in_v) y = *reinterpret_cast<const float2*>(p + v_off + h * vdim + 2 * i);
      store_pair<T>(v_dst + h * head_stride + 2 * i, y.x, y.y);
    }
  }
}

// The same step for layers that normalise their queries and keys: every query and key head is divided by its root
// mean square over `dim` (eps inside the root) and multiplied by a weight of `dim` values that all heads share
// (wq for queries, wk for keys; null: no norm for that kind), then turned by the position as above, cast, padded and
// written.  A warp owns a head; lane l owns the pairs l, l + 32, ... of it (at most four: dim <= 256).
template <typename T>
__global__ void __launch_bounds__(256)
norm_rope_append_kernel(const float* proj, int ld, int q_off, int k_off, int v_off, int n_head, int n_kv_head, int dim,
                        int vdim, int hd, const float* __restrict__ wq, const float* __restrict__ wk, float eps,
                        int rot_dims, const double* __restrict__ freqs, const int* __restrict__ positions,
                        const int* __restrict__ row_entry, T* q_out, int ldq, T* cache,
                        const int* __restrict__ block_table, int max_blocks, int page_size, int n_pages, int* status) {
  pdl_trigger();
  const int t = blockIdx.y, lane = threadIdx.x & 31;
  const int hh = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (hh >= n_head + 2 * n_kv_head) return;
  const int pos = positions[t], entry = row_entry[t];
  const bool is_q = hh < n_head, is_k = !is_q && hh < n_head + n_kv_head;
  const int h = is_q ? hh : (is_k ? hh - n_head : hh - n_head - n_kv_head);
  T* dst = nullptr;
  if (is_q) {
    dst = q_out + (size_t)t * ldq + (size_t)h * hd;
  } else if (entry >= 0 && cache != nullptr) {
    const int page = block_table[(size_t)entry * max_blocks + pos / page_size];
    if (page < 0 || page >= n_pages) {
      if (lane == 0) *status = NIB_STATUS_BAD_PAGE;
    } else {
      dst = cache + kv_offset(page, is_k ? 0 : 1, h, pos % page_size, n_kv_head, page_size, hd);
    }
  }
  pdl_wait();
  if (dst == nullptr) return;
  const int width = is_q || is_k ? dim : vdim;
  const float* src = proj + (size_t)t * ld + (is_q ? q_off : (is_k ? k_off : v_off)) + (size_t)h * width;
  const float* w = is_q ? wq : (is_k ? wk : nullptr);
  float2 x[4];
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = 2 * (lane + 32 * i);
    x[i] = c < width ? *reinterpret_cast<const float2*>(src + c) : make_float2(0.0f, 0.0f);
    ss += x[i].x * x[i].x + x[i].y * x[i].y;
  }
  float r = 1.0f;
  if (w != nullptr) r = 1.0f / sqrtf(warp_sum(ss) / (float)width + eps);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = 2 * (lane + 32 * i);
    if (c >= hd) continue;
    float u = 0.0f, v = 0.0f;
    if (c < width) {
      u = x[i].x * r;
      v = x[i].y * r;
      if (w != nullptr) {
        u *= w[c];
        v *= w[c + 1];
      }
      if ((is_q || is_k) && c < rot_dims) {
        double sd, cd;
        sincos((double)pos * freqs[c >> 1], &sd, &cd);
        const float cs = (float)cd, sn = (float)sd, a = u, b = v;
        u = a * cs - b * sn;
        v = b * cs + a * sn;
      }
    }
    store_pair<T>(dst + c, u, v);
  }
}

}  // namespace nib

using namespace nib;

// dim, vdim, hd, rot_dims, ld, ldq and the three offsets even; rot_dims <= dim <= hd, vdim <= hd; freqs holds
// rot_dims / 2 values (may be null when rot_dims is 0); cache may be null (queries only).
extern "C" int nib_rope_append(int dtype, const float* proj, int ld, int q_off, int k_off, int v_off, int n_head,
                               int n_kv_head, int dim, int vdim, int hd, int rot_dims, const double* freqs,
                               const int* positions, const int* row_entry, void* q_out, int ldq, void* cache,
                               const int* block_table, int max_blocks, int page_size, int n_pages, int T, int* status,
                               cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((dim | vdim | hd | rot_dims | ld | ldq | q_off | k_off | v_off) & 1) return NIB_ERR_UNSUPPORTED_SIZE;
  if (dim <= 0 || vdim <= 0 || dim > hd || vdim > hd || rot_dims < 0 || rot_dims > dim) return NIB_ERR_BAD_ARGUMENT;
  if (rot_dims > 0 && freqs == nullptr) return NIB_ERR_BAD_ARGUMENT;
  if (hd / 2 > 256) return NIB_ERR_UNSUPPORTED_SIZE;
  const int per = hd / 2, total = n_head + 2 * n_kv_head;
  int groups = 256 / per;
  if (groups > total) groups = total;
  const dim3 block(groups * per);
  if (dtype == DT_F32)
    launch_pdl(rope_append_kernel<float>, dim3(T), block, 0, stream, proj, ld, q_off, k_off, v_off, n_head, n_kv_head,
               dim, vdim, hd, rot_dims, freqs, positions, row_entry, (float*)q_out, ldq, (float*)cache, block_table,
               max_blocks, page_size, n_pages, status);
  else if (dtype == DT_BF16)
    launch_pdl(rope_append_kernel<bf16>, dim3(T), block, 0, stream, proj, ld, q_off, k_off, v_off, n_head, n_kv_head,
               dim, vdim, hd, rot_dims, freqs, positions, row_entry, (bf16*)q_out, ldq, (bf16*)cache, block_table,
               max_blocks, page_size, n_pages, status);
  else
    return NIB_ERR_BAD_ARGUMENT;
  NIB_LAUNCH_CHECK();
}

// The same with a norm of every query and key head ahead of the rotation (norm_rope_append_kernel): wq and wk hold
// `dim` values each (either may be null); hd <= 256.
extern "C" int nib_norm_rope_append(int dtype, const float* proj, int ld, int q_off, int k_off, int v_off, int n_head,
                                    int n_kv_head, int dim, int vdim, int hd, const float* wq, const float* wk,
                                    float eps, int rot_dims, const double* freqs, const int* positions,
                                    const int* row_entry, void* q_out, int ldq, void* cache, const int* block_table,
                                    int max_blocks, int page_size, int n_pages, int T, int* status,
                                    cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((dim | vdim | hd | rot_dims | ld | ldq | q_off | k_off | v_off) & 1) return NIB_ERR_UNSUPPORTED_SIZE;
  if (dim <= 0 || vdim <= 0 || dim > hd || vdim > hd || rot_dims < 0 || rot_dims > dim) return NIB_ERR_BAD_ARGUMENT;
  if (rot_dims > 0 && freqs == nullptr) return NIB_ERR_BAD_ARGUMENT;
  if (hd > 256 || T > 65535) return NIB_ERR_UNSUPPORTED_SIZE;
  const int total = n_head + 2 * n_kv_head;
  const int warps = total < 8 ? total : 8;
  const dim3 grid((total + warps - 1) / warps, T), block(32 * warps);
  if (dtype == DT_F32)
    launch_pdl(norm_rope_append_kernel<float>, grid, block, 0, stream, proj, ld, q_off, k_off, v_off, n_head, n_kv_head,
               dim, vdim, hd, wq, wk, eps, rot_dims, freqs, positions, row_entry, (float*)q_out, ldq, (float*)cache,
               block_table, max_blocks, page_size, n_pages, status);
  else if (dtype == DT_BF16)
    launch_pdl(norm_rope_append_kernel<bf16>, grid, block, 0, stream, proj, ld, q_off, k_off, v_off, n_head, n_kv_head,
               dim, vdim, hd, wq, wk, eps, rot_dims, freqs, positions, row_entry, (bf16*)q_out, ldq, (bf16*)cache,
               block_table, max_blocks, page_size, n_pages, status);
  else
    return NIB_ERR_BAD_ARGUMENT;
  NIB_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------------------------
// The halves layout: of a head's first `rot_dims` values, value i is paired with value i + rot_dims / 2 and the
// pair (u, w) at position p becomes (u cos a - w sin a, w cos a + u sin a), a = p * freqs[i]; the other values pass.
namespace nib {

// Queries and keys normed over the WHOLE projection (all heads at once: x / sqrt(mean(x^2) + eps) times a weight of
// the projection's size; null: no norm), then turned in the halves layout, cast, padded to the cache's head size and
// written: queries to q_out, keys to plane 0 of the row's cache slot; plane 1 receives the values, which are read as
// they stand (v_off may name the keys' own columns: a layer whose values are its keys ahead of norm and rotation).
// A block a row.
template <typename T>
__global__ void __launch_bounds__(256)
wide_norm_rope_append_kernel(const float* src, int ld, int q_off, int k_off, int v_off, int n_head, int n_kv_head,
                             int dim, int vdim, int hd, const float* __restrict__ wq, const float* __restrict__ wk,
                             float eps, int rot_dims, const double* __restrict__ freqs,
                             const int* __restrict__ positions, const int* __restrict__ row_entry, T* q_out, int ldq,
                             T* cache, const int* __restrict__ block_table, int max_blocks, int page_size, int n_pages,
                             int* status) {
  pdl_trigger();
  extern __shared__ float cs[];          // [rot_dims / 2] cosines, then as many sines
  __shared__ float scratch[32];
  const int t = blockIdx.x, half = rot_dims / 2;
  const int pos = positions[t], entry = row_entry[t];
  float* sn = cs + half;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    double sd, cd;
    sincos((double)pos * freqs[i], &sd, &cd);
    cs[i] = (float)cd;
    sn[i] = (float)sd;
  }
  T* k_dst = nullptr;
  T* v_dst = nullptr;
  if (entry >= 0 && cache != nullptr) {
    const int page = block_table[(size_t)entry * max_blocks + pos / page_size];
    if (page < 0 || page >= n_pages) {
      if (threadIdx.x == 0) *status = NIB_STATUS_BAD_PAGE;
    } else {
      k_dst = cache + kv_offset(page, 0, 0, pos % page_size, n_kv_head, page_size, hd);
      v_dst = cache + kv_offset(page, 1, 0, pos % page_size, n_kv_head, page_size, hd);
    }
  }
  const size_t head_stride = (size_t)page_size * hd;
  pdl_wait();
  const float* p = src + (size_t)t * ld;
  const int nq = n_head * dim, nk = n_kv_head * dim;
  float sq = 0.0f, sk = 0.0f;
  if (wq != nullptr)
    for (int i = threadIdx.x; i < nq; i += blockDim.x) sq += p[q_off + i] * p[q_off + i];
  if (wk != nullptr && k_dst != nullptr)
    for (int i = threadIdx.x; i < nk; i += blockDim.x) sk += p[k_off + i] * p[k_off + i];
  const float rq = wq != nullptr ? 1.0f / sqrtf(block_sum(sq, scratch) / (float)nq + eps) : 1.0f;
  const float rk = wk != nullptr ? 1.0f / sqrtf(block_sum(sk, scratch) / (float)nk + eps) : 1.0f;
  __syncthreads();
  const int n_rot = (n_head + (k_dst != nullptr ? n_kv_head : 0)) * hd;
  for (int idx = threadIdx.x; idx < n_rot; idx += blockDim.x) {
    const int hh = idx / hd, c = idx % hd;
    const bool is_q = hh < n_head;
    const int h = is_q ? hh : hh - n_head;
    const float* x = p + (is_q ? q_off : k_off) + h * dim;
    const float* w = is_q ? wq : wk;
    const float r = is_q ? rq : rk;
    float v = 0.0f;
    if (c < dim) {
      v = x[c] * r;
      if (w != nullptr) v *= w[h * dim + c];
      if (c < rot_dims) {
        const int pc = c < half ? c + half : c - half, i = c < half ? c : c - half;
        float o = x[pc] * r;
        if (w != nullptr) o *= w[h * dim + pc];
        v = c < half ? v * cs[i] - o * sn[i] : v * cs[i] + o * sn[i];
      }
    }
    if (is_q) q_out[(size_t)t * ldq + (size_t)h * hd + c] = from_float<T>(v);
    else k_dst[h * head_stride + c] = from_float<T>(v);
  }
  if (v_dst != nullptr)
    for (int idx = threadIdx.x; idx < n_kv_head * hd; idx += blockDim.x) {
      const int h = idx / hd, c = idx % hd;
      v_dst[h * head_stride + c] = from_float<T>(c < vdim ? p[v_off + h * vdim + c] : 0.0f);
    }
}

// In place on 32-bit rows: the query and key heads (n_head of `dim` values each at q_off and at k_off) turned in the
// halves layout, the keys then times k_mul; and coef[t, h] = (decay[h], 1): what a recurrence with one fixed decay
// per head reads as its rows' decays and strengths.  A block a row; a thread owns a pair (or a value that passes).
__global__ void __launch_bounds__(256)
rope_halves_kernel(float* rows, int ld, int q_off, int k_off, int n_head, int dim, int rot_dims,
                   const double* __restrict__ freqs, const int* __restrict__ positions, float k_mul,
                   const float* __restrict__ decay, float* coef) {
  pdl_trigger();
  extern __shared__ float cs[];
  const int t = blockIdx.x, half = rot_dims / 2;
  const int pos = positions[t];
  float* sn = cs + half;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    double sd, cd;
    sincos((double)pos * freqs[i], &sd, &cd);
    cs[i] = (float)cd;
    sn[i] = (float)sd;
  }
  __syncthreads();
  pdl_wait();
  // (nothing is written ahead of the wait: a kernel further back may still be reading coef, which layers share)
  if (coef != nullptr)
    for (int h = threadIdx.x; h < n_head; h += blockDim.x) {
      coef[((size_t)t * n_head + h) * 2] = decay[h];
      coef[((size_t)t * n_head + h) * 2 + 1] = 1.0f;
    }
  float* p = rows + (size_t)t * ld;
  const int units = dim - half;            // per head: `half` pairs, then the values behind rot_dims
  for (int idx = threadIdx.x; idx < 2 * n_head * units; idx += blockDim.x) {
    const int hh = idx / units, u = idx % units;
    const bool is_q = hh < n_head;
    float* x = p + (is_q ? q_off : k_off) + (is_q ? hh : hh - n_head) * dim;
    const float mul = is_q ? 1.0f : k_mul;
    if (u < half) {
      const float a = x[u], b = x[u + half];
      x[u] = (a * cs[u] - b * sn[u]) * mul;
      x[u + half] = (b * cs[u] + a * sn[u]) * mul;
    } else {
      x[u + half] *= mul;
    }
  }
}

}  // namespace nib

extern "C" int nib_wide_norm_rope_append(int dtype, const float* src, int ld, int q_off, int k_off, int v_off,
                                         int n_head, int n_kv_head, int dim, int vdim, int hd, const float* wq,
                                         const float* wk, float eps, int rot_dims, const double* freqs,
                                         const int* positions, const int* row_entry, void* q_out, int ldq, void* cache,
                                         const int* block_table, int max_blocks, int page_size, int n_pages, int T,
                                         int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (dim <= 0 || vdim <= 0 || dim > hd || vdim > hd || rot_dims < 0 || rot_dims > dim || (rot_dims & 1))
    return NIB_ERR_BAD_ARGUMENT;
  if (rot_dims > 0 && freqs == nullptr) return NIB_ERR_BAD_ARGUMENT;
  const size_t smem = (size_t)rot_dims * sizeof(float);
  if (smem > 48 * 1024) return NIB_ERR_UNSUPPORTED_SIZE;
  if (dtype == DT_F32)
    launch_pdl(wide_norm_rope_append_kernel<float>, dim3(T), dim3(256), smem, stream, src, ld, q_off, k_off, v_off,
               n_head, n_kv_head, dim, vdim, hd, wq, wk, eps, rot_dims, freqs, positions, row_entry, (float*)q_out, ldq,
               (float*)cache, block_table, max_blocks, page_size, n_pages, status);
  else if (dtype == DT_BF16)
    launch_pdl(wide_norm_rope_append_kernel<bf16>, dim3(T), dim3(256), smem, stream, src, ld, q_off, k_off, v_off,
               n_head, n_kv_head, dim, vdim, hd, wq, wk, eps, rot_dims, freqs, positions, row_entry, (bf16*)q_out, ldq,
               (bf16*)cache, block_table, max_blocks, page_size, n_pages, status);
  else
    return NIB_ERR_BAD_ARGUMENT;
  NIB_LAUNCH_CHECK();
}

extern "C" int nib_rope_halves(float* rows, int ld, int q_off, int k_off, int n_head, int dim, int rot_dims,
                               const double* freqs, const int* positions, float k_mul, const float* decay, float* coef,
                               int T, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (dim <= 0 || rot_dims < 0 || rot_dims > dim || (rot_dims & 1) || (rot_dims > 0 && freqs == nullptr) ||
      (coef != nullptr && decay == nullptr))
    return NIB_ERR_BAD_ARGUMENT;
  const size_t smem = (size_t)rot_dims * sizeof(float);
  if (smem > 48 * 1024) return NIB_ERR_UNSUPPORTED_SIZE;
  launch_pdl(rope_halves_kernel, dim3(T), dim3(256), smem, stream, rows, ld, q_off, k_off, n_head, dim, rot_dims, freqs,
             positions, k_mul, decay, coef);
  NIB_LAUNCH_CHECK();
}
