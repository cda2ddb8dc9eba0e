// The selective scan of Mamba: per channel c of the inner width and state index n, with the row's step size
// dt_c = softplus(dtp_c), its input x_c, and the row's vectors B and C (shared by all channels):
//   S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n;    y_c = sum_n S[c, n] C_n + D_c x_c;    out_c = y_c silu(z_c)
// with A = -exp(A_log).  S starts at zero, lives in 32-bit floats in the request's state slot and is carried from
// row to row of the request; step sizes, decays, the recurrence and the gate are 32-bit.
//
// Channels do not see one another.  A channel is owned by L neighbouring lanes (L a power of two, at most 32); lane j
// of them keeps the states n = j, j + L, ... (PER of them: 1, 2, 4 or 8) and A's values for them in registers, and the
// read-out's sum over n ends with log2(L) shuffles.  A block of 128 threads owns 128 / L channels of one batch entry
// and walks the entry's rows in order, SSM_ROWS rows at a time through a double buffer in shared memory filled by
// cp.async: the rows' B and C, and for the block's channels dtp and z (turned into softplus(dtp) and silu(z) once
// they have landed) and x.  Of a chunk's rows the decays (less one) and the inputs dt x B are made first, side by side; only the
// multiply-adds into S form a chain from row to row, and the read-outs' sums are taken off it afterwards.
//
// State per request: [inner][NP] floats with NP = L * PER; the entries behind N stay zero.
//
// The decay enters as exp(dt A) - 1 (ssm_expm1 below) and the update is S <- S + (decay - 1) S + input: a channel that
// forgets slowly has a decay next to 1, whose 32-bit value carries the little that is forgotten with three or four
// digits only, the same way at every row, and over a prompt of a thousand rows that error in what is remembered of
// the first rows grows with the distance (measured: the 32-bit model's error against a float64 one grew in
// proportion to the position with exp(dt A) and stays flat with this form; carrying S in double precision on top
// changes nothing more).
#include "api.h"
#include "common.cuh"

namespace nib {

constexpr int SSM_THREADS = 128;
constexpr int SSM_ROWS = 8;      // rows staged at a time

__device__ __forceinline__ float ssm_softplus(float v) { return v > 20.0f ? v : log1pf(expf(v)); }

// exp(z) - 1 for z <= 0.  Below 1/16 the series up to z^6 (its next term is under 2^-36 of z); from there on
// exp(z) - 1, whose one part in 2^24 of exp(z) is then under a part in 2^20 of what is forgotten, in channels whose
// memory is a few hundred rows at most.
__device__ __forceinline__ float ssm_expm1(float z) {
  const float p = z * fmaf(z, fmaf(z, fmaf(z, fmaf(z, fmaf(z, 1.0f / 720.0f, 1.0f / 120.0f), 1.0f / 24.0f), 1.0f / 6.0f), 0.5f), 1.0f);
  return fabsf(z) < 0.0625f ? p : expf(z) - 1.0f;
}

__device__ __forceinline__ void ssm_cp4(void* smem_dst, const void* gmem_src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(gmem_src) : "memory");
}

// the states a lane keeps (1, 2, 4 or 8) and the lanes of a channel for a state of N values: two states a lane while
// the lanes of a warp suffice, more beyond
static inline void ssm_shape(int N, int* L, int* PER) {
  int l = 1;
  while (l < 32 && (N + l - 1) / l > 2) l <<= 1;
  int per = 1;
  while (per * l < N) per <<= 1;
  *L = l;
  *PER = per;
}

// dtp [T, ld_dt]: the step sizes before the softplus (bias included); x [T, ldx]: the channels' inputs;
// bc [T, ldbc]: B at b_off, C at c_off (N values each); z [T, ldz]: the gates' inputs; out [T, ldo].
template <typename OutT, int PER>
__global__ void __launch_bounds__(SSM_THREADS)
selective_scan_kernel(const float* dtp, int ld_dt, const float* x, int ldx, const float* bc, int ldbc, int b_off,
                      int c_off, const float* z, int ldz, const float* __restrict__ A_log, const float* __restrict__ D,
                      float* state, long long state_stride, long long s_off, const int* __restrict__ entry_start,
                      const int* __restrict__ entry_slot, int inner, int N, int L, OutT* out, int ldo) {
  pdl_trigger();
  extern __shared__ float sm[];
  const int NP = PER * L, CH = SSM_THREADS / L;
  const int BUF = SSM_ROWS * (2 * NP + 3 * CH);          // per buffer: B | C | dt | x | z
  const int e = blockIdx.y, tid = threadIdx.x, j = tid % L, cl = tid / L;
  const int c = blockIdx.x * CH + cl;
  const bool has = c < inner;
  const int r0 = entry_start[e], n_rows = entry_start[e + 1] - r0;
  float a[PER], S[PER];
  float* sp = state + (size_t)entry_slot[e] * state_stride + s_off + (size_t)(has ? c : 0) * NP;
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    const int n = j + k * L;
    a[k] = (has && n < N) ? -expf(A_log[(size_t)c * N + n]) : 0.0f;
    // the state belongs to this kernel alone: what it holds was written a step ago
    S[k] = has ? sp[n] : 0.0f;
  }
  const float d_skip = has ? D[c] : 0.0f;
  for (int i = tid; i < 2 * BUF; i += SSM_THREADS) sm[i] = 0.0f;   // (the tails behind N and the inner width stay zero)
  __syncthreads();
  pdl_wait();

  // asks for the rows of chunk ck into buffer b
  auto stage = [&](int ck, int b) {
    float* sB = sm + b * BUF;
    float* sC = sB + SSM_ROWS * NP;
    float* sdt = sC + SSM_ROWS * NP;
    float* sx = sdt + SSM_ROWS * CH;
    float* sz = sx + SSM_ROWS * CH;
    const int rows = min(SSM_ROWS, n_rows - ck * SSM_ROWS);
    for (int i = tid; i < rows * N; i += SSM_THREADS) {
      const int rr = i / N, n = i % N;
      const float* src = bc + (size_t)(r0 + ck * SSM_ROWS + rr) * ldbc;
      ssm_cp4(sB + rr * NP + n, src + b_off + n);
      ssm_cp4(sC + rr * NP + n, src + c_off + n);
    }
    for (int i = tid; i < rows * CH; i += SSM_THREADS) {
      const int rr = i / CH, cc = blockIdx.x * CH + i % CH;
      if (cc < inner) {
        const size_t t = r0 + ck * SSM_ROWS + rr;
        ssm_cp4(sdt + i, dtp + t * ld_dt + cc);
        ssm_cp4(sx + i, x + t * ldx + cc);
        ssm_cp4(sz + i, z + t * ldz + cc);
      }
    }
    cp_async_commit();
  };

  const int n_chunks = (n_rows + SSM_ROWS - 1) / SSM_ROWS;
  if (n_chunks > 0) stage(0, 0);
  for (int ck = 0; ck < n_chunks; ++ck) {
    cp_async_wait<0>();
    __syncthreads();   // chunk ck has arrived, and every thread is done with the buffer that chunk ck + 1 goes to
    if (ck + 1 < n_chunks) stage(ck + 1, (ck + 1) & 1);
    const int rows = min(SSM_ROWS, n_rows - ck * SSM_ROWS);
    float* sB = sm + (ck & 1) * BUF;
    float* sC = sB + SSM_ROWS * NP;
    float* sdt = sC + SSM_ROWS * NP;
    const float* sx = sdt + SSM_ROWS * CH;
    float* sz = sdt + 2 * SSM_ROWS * CH;
    for (int i = tid; i < rows * CH; i += SSM_THREADS) {   // each step size and each gate once
      sdt[i] = ssm_softplus(sdt[i]);
      const float zv = sz[i];
      sz[i] = zv / (1.0f + expf(-zv));
    }
    __syncthreads();
    // (lanes of channels beyond the inner width walk along with zeros: the shuffles below want whole warps)
    float da[SSM_ROWS][PER], db[SSM_ROWS][PER], acc[SSM_ROWS];
#pragma unroll
    for (int rr = 0; rr < SSM_ROWS; ++rr) {
      const float dt = rr < rows ? sdt[rr * CH + cl] : 0.0f;
      const float dx = rr < rows ? dt * sx[rr * CH + cl] : 0.0f;
#pragma unroll
      for (int k = 0; k < PER; ++k) {
        da[rr][k] = ssm_expm1(dt * a[k]);   // the decay less one: what a slow channel forgets is all of its decay's information
        db[rr][k] = dx * sB[rr * NP + j + k * L];
      }
    }
#pragma unroll
    for (int rr = 0; rr < SSM_ROWS; ++rr) {
      float t = 0.0f;
      if (rr < rows) {
#pragma unroll
        for (int k = 0; k < PER; ++k) {
          S[k] = fmaf(da[rr][k], S[k], S[k]) + db[rr][k];     // S + (decay - 1) S + input
          t = fmaf(S[k], sC[rr * NP + j + k * L], t);
        }
      }
      acc[rr] = t;
    }
#pragma unroll
    for (int rr = 0; rr < SSM_ROWS; ++rr) {
      float t = acc[rr];
      for (int o = 1; o < L; o <<= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
      if (rr < rows && j == 0 && has) {
        const float y = fmaf(d_skip, sx[rr * CH + cl], t);
        out[(size_t)(r0 + ck * SSM_ROWS + rr) * ldo + c] = from_float<OutT>(y * sz[rr * CH + cl]);
      }
    }
  }
  if (has) {
#pragma unroll
    for (int k = 0; k < PER; ++k) sp[j + k * L] = S[k];
  }
}

template <typename OutT>
static int launch_ssm(dim3 grid, size_t smem, cudaStream_t stream, int PER, const float* dtp, int ld_dt, const float* x,
                      int ldx, const float* bc, int ldbc, int b_off, int c_off, const float* z, int ldz,
                      const float* A_log, const float* D, float* state, long long state_stride, long long s_off,
                      const int* entry_start, const int* entry_slot, int inner, int N, int L, OutT* out, int ldo) {
#define NIB_SSM(P)                                                                                                      \
  launch_pdl(selective_scan_kernel<OutT, P>, grid, dim3(SSM_THREADS), smem, stream, dtp, ld_dt, x, ldx, bc, ldbc, b_off, \
             c_off, z, ldz, A_log, D, state, state_stride, s_off, entry_start, entry_slot, inner, N, L, out, ldo)
  if (PER == 1) NIB_SSM(1);
  else if (PER == 2) NIB_SSM(2);
  else if (PER == 4) NIB_SSM(4);
  else NIB_SSM(8);
#undef NIB_SSM
  NIB_LAUNCH_CHECK();
}

}  // namespace nib

using namespace nib;

// Floats of state that one request's selective scan keeps: [inner][N rounded up to lanes x states a lane]
// (0: N is too large).
extern "C" long long nib_selective_scan_state_floats(int inner, int N) {
  if (N <= 0 || N > 256) return 0;
  int L, PER;
  ssm_shape(N, &L, &PER);
  return (long long)inner * L * PER;
}

extern "C" int nib_selective_scan(int out_dtype, const float* dtp, int ld_dt, const float* x, int ldx, const float* bc,
                                  int ldbc, int b_off, int c_off, const float* z, int ldz, const float* A_log,
                                  const float* D, float* state, long long state_stride, long long s_off,
                                  const int* entry_start, const int* entry_slot, int n_entries, int inner, int N,
                                  void* out, int ldo, cudaStream_t stream) {
  if (n_entries <= 0) return 0;
  if (inner <= 0 || N <= 0 || N > 256 || n_entries > 65535) return NIB_ERR_UNSUPPORTED_SIZE;
  int L, PER;
  ssm_shape(N, &L, &PER);
  const int CH = SSM_THREADS / L, NP = L * PER;
  const size_t smem = (size_t)2 * SSM_ROWS * (2 * NP + 3 * CH) * sizeof(float);
  const dim3 grid((inner + CH - 1) / CH, n_entries);
  if (out_dtype == DT_F32)
    return launch_ssm<float>(grid, smem, stream, PER, dtp, ld_dt, x, ldx, bc, ldbc, b_off, c_off, z, ldz, A_log, D, state,
                             state_stride, s_off, entry_start, entry_slot, inner, N, L, (float*)out, ldo);
  if (out_dtype == DT_BF16)
    return launch_ssm<bf16>(grid, smem, stream, PER, dtp, ld_dt, x, ldx, bc, ldbc, b_off, c_off, z, ldz, A_log, D, state,
                            state_stride, s_off, entry_start, entry_slot, inner, N, L, (bf16*)out, ldo);
  return NIB_ERR_BAD_ARGUMENT;
}
