// The selective scan of Mamba: per channel c of the inner width and state index n, with the row's step size
// dt_c = softplus(dtp_c), its input x_c, and the row's vectors B and C (shared by all channels):
//   S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n;    y_c = sum_n S[c, n] C_n + D_c x_c;    out_c = y_c silu(z_c)
// with A = -exp(A_log).  S starts at zero, lives in 32-bit floats in the request's state slot and is carried from
// row to row of the request; step sizes, decays, the recurrence and the gate are 32-bit.
//
// Channels do not see one another.  A channel is owned by L neighbouring lanes (L a power of two, at most 32); lane j
// of them keeps the states n = j, j + L, ... (at most SSM_PER) and A's values for them in registers, and the
// read-out's sum over n ends with log2(L) shuffles.  A block of 128 threads owns 128 / L channels of one batch entry
// and walks the entry's rows in order, SSM_ROWS rows staged into shared memory at a time: the rows' B and C, and
// for the block's channels softplus(dtp), x and z.
//
// State per request: [inner][NP] floats with NP = L * ceil(N / L); the entries behind N stay zero.
#include "api.h"
#include "common.cuh"

namespace nib {

constexpr int SSM_THREADS = 128;
constexpr int SSM_PER = 8;       // states per lane at most
constexpr int SSM_ROWS = 8;      // rows staged at a time

__device__ __forceinline__ float ssm_softplus(float v) { return v > 20.0f ? v : log1pf(expf(v)); }

// the lanes of a channel for a state of N values: the smallest power of two with ceil(N / L) <= SSM_PER
static inline int ssm_lanes(int N) {
  int L = 1;
  while ((N + L - 1) / L > SSM_PER) L <<= 1;
  return L;
}

// dtp [T, ld_dt]: the step sizes before the softplus (bias included); x [T, ldx]: the channels' inputs;
// bc [T, ldbc]: B at b_off, C at c_off (N values each); z [T, ldz]: the gates' inputs; out [T, ldo].
template <typename OutT>
__global__ void __launch_bounds__(SSM_THREADS)
selective_scan_kernel(const float* dtp, int ld_dt, const float* x, int ldx, const float* bc, int ldbc, int b_off,
                      int c_off, const float* z, int ldz, const float* __restrict__ A_log, const float* __restrict__ D,
                      float* state, long long state_stride, long long s_off, const int* __restrict__ entry_start,
                      const int* __restrict__ entry_slot, int inner, int N, int L, OutT* out, int ldo) {
  pdl_trigger();
  extern __shared__ float sm[];
  const int per = (N + L - 1) / L, NP = per * L, CH = SSM_THREADS / L;
  float* sB = sm;                               // [SSM_ROWS][NP]
  float* sC = sB + SSM_ROWS * NP;               // [SSM_ROWS][NP]
  float* sdt = sC + SSM_ROWS * NP;              // [SSM_ROWS][CH]
  float* sx = sdt + SSM_ROWS * CH;              // [SSM_ROWS][CH]
  float* sz = sx + SSM_ROWS * CH;               // [SSM_ROWS][CH]
  const int e = blockIdx.y, tid = threadIdx.x, j = tid % L, cl = tid / L;
  const int c = blockIdx.x * CH + cl;
  const bool has = c < inner;
  const int r0 = entry_start[e], n_rows = entry_start[e + 1] - r0;
  float a[SSM_PER], S[SSM_PER];
  float* sp = state + (size_t)entry_slot[e] * state_stride + s_off + (size_t)(has ? c : 0) * NP;
#pragma unroll
  for (int k = 0; k < SSM_PER; ++k) {
    const int n = j + k * L;
    a[k] = (has && k < per && n < N) ? -expf(A_log[(size_t)c * N + n]) : 0.0f;
    S[k] = 0.0f;
  }
  const float d_skip = has ? D[c] : 0.0f;
  for (int i = tid; i < 2 * SSM_ROWS * NP; i += SSM_THREADS) sm[i] = 0.0f;   // (the tails behind N stay zero)
  // the state belongs to this kernel alone: what it holds was written a step ago
#pragma unroll
  for (int k = 0; k < SSM_PER; ++k)
    if (has && k < per) S[k] = sp[j + k * L];
  pdl_wait();
  for (int base = 0; base < n_rows; base += SSM_ROWS) {
    const int rows = min(SSM_ROWS, n_rows - base);
    __syncthreads();     // everyone is done with the rows staged before
    for (int i = tid; i < rows * N; i += SSM_THREADS) {
      const int rr = i / N, n = i % N;
      const float* src = bc + (size_t)(r0 + base + rr) * ldbc;
      sB[rr * NP + n] = src[b_off + n];
      sC[rr * NP + n] = src[c_off + n];
    }
    for (int i = tid; i < rows * CH; i += SSM_THREADS) {
      const int rr = i / CH, cc = blockIdx.x * CH + i % CH;
      if (cc < inner) {
        const size_t t = r0 + base + rr;
        sdt[i] = ssm_softplus(dtp[t * ld_dt + cc]);
        sx[i] = x[t * ldx + cc];
        sz[i] = z[t * ldz + cc];
      }
    }
    __syncthreads();
    // (lanes of channels beyond the inner width walk along with zeros: the shuffles below want whole warps)
    for (int rr = 0; rr < rows; ++rr) {
      const float dt = sdt[rr * CH + cl], xv = sx[rr * CH + cl];
      const float dx = dt * xv;
      const float* Br = sB + rr * NP;
      const float* Cr = sC + rr * NP;
      float acc = 0.0f;
#pragma unroll
      for (int k = 0; k < SSM_PER; ++k) {
        if (k < per) {
          S[k] = fmaf(expf(dt * a[k]), S[k], dx * Br[j + k * L]);
          acc = fmaf(S[k], Cr[j + k * L], acc);
        }
      }
      for (int o = 1; o < L; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (j == 0 && has) {
        const float zv = sz[rr * CH + cl];
        const float y = fmaf(d_skip, xv, acc);
        out[(size_t)(r0 + base + rr) * ldo + c] = from_float<OutT>(y * (zv / (1.0f + expf(-zv))));
      }
    }
  }
  if (has) {
#pragma unroll
    for (int k = 0; k < SSM_PER; ++k)
      if (k < per) sp[j + k * L] = S[k];
  }
}

}  // namespace nib

using namespace nib;

// Floats of state that one request's selective scan keeps: [inner][N rounded up to the lanes of a channel]
// (0: N is too large).
extern "C" long long nib_selective_scan_state_floats(int inner, int N) {
  if (N <= 0 || N > 32 * SSM_PER) return 0;
  const int L = ssm_lanes(N);
  return (long long)inner * ((N + L - 1) / L) * L;
}

extern "C" int nib_selective_scan(int out_dtype, const float* dtp, int ld_dt, const float* x, int ldx, const float* bc,
                                  int ldbc, int b_off, int c_off, const float* z, int ldz, const float* A_log,
                                  const float* D, float* state, long long state_stride, long long s_off,
                                  const int* entry_start, const int* entry_slot, int n_entries, int inner, int N,
                                  void* out, int ldo, cudaStream_t stream) {
  if (n_entries <= 0) return 0;
  if (inner <= 0 || N <= 0 || N > 32 * SSM_PER || n_entries > 65535) return NIB_ERR_UNSUPPORTED_SIZE;
  const int L = ssm_lanes(N), CH = SSM_THREADS / L, NP = (N + L - 1) / L * L;
  const size_t smem = (size_t)(2 * SSM_ROWS * NP + 3 * SSM_ROWS * CH) * sizeof(float);
  const dim3 grid((inner + CH - 1) / CH, n_entries);
  if (out_dtype == DT_F32)
    launch_pdl(selective_scan_kernel<float>, grid, dim3(SSM_THREADS), smem, stream, dtp, ld_dt, x, ldx, bc, ldbc, b_off,
               c_off, z, ldz, A_log, D, state, state_stride, s_off, entry_start, entry_slot, inner, N, L, (float*)out, ldo);
  else if (out_dtype == DT_BF16)
    launch_pdl(selective_scan_kernel<bf16>, grid, dim3(SSM_THREADS), smem, stream, dtp, ld_dt, x, ldx, bc, ldbc, b_off,
               c_off, z, ldz, A_log, D, state, state_stride, s_off, entry_start, entry_slot, inner, N, L, (bf16*)out, ldo);
  else
    return NIB_ERR_BAD_ARGUMENT;
  NIB_LAUNCH_CHECK();
}
