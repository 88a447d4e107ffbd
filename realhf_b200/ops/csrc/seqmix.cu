// Row-wise mechanisms of heterogeneous stacks: grouped RMSNorm fused with a short causal convolution over time (packed and
// one-token forms, the latter with its per-sequence state), residual add fused with a grouped RMSNorm of the branch output,
// the clamped gated-linear-unit activation and the soft cap on logits.
//
// All arithmetic is fp32 whatever the storage types: TX is the residual stream's type (fp32 when the model keeps an fp32
// residual), TA the activation / weight type.  One CTA per row; a (row, group) root mean square is reduced by ONE warp in a
// fixed order, so results do not depend on the batch a row is in.  Compiled without fast-math.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kMaxTaps = 8;

RB_DEVICE float ld_any(const void* p, int dt, int64_t i) {
  if (dt == 0) return static_cast<const float*>(p)[i];
  if (dt == 1) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(static_cast<const __half*>(p)[i]);
}
RB_DEVICE void st_any(void* p, int dt, int64_t i, float v) {
  if (dt == 0) static_cast<float*>(p)[i] = v;
  else if (dt == 1) static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else static_cast<__half*>(p)[i] = __float2half_rn(v);
}

// rstd[r * groups + g] for `n_rows` source rows (row r at x + row_off[r] * W, skipped when row_off[r] < 0): warp w takes the
// (row, group) pairs w, w + nwarps, ...
RB_DEVICE void group_rstd(const void* x, int dtx, const int64_t* row_off, int n_rows, int W, int groups, float eps, float* rstd) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int gs = W / groups;
  for (int pair = warp; pair < n_rows * groups; pair += nwarp) {
    const int r = pair / groups, g = pair % groups;
    if (row_off[r] < 0) continue;
    const int64_t base = row_off[r] * (int64_t)W + (int64_t)g * gs;
    float s = 0.f;
    for (int e = lane; e < gs; e += 32) { const float v = ld_any(x, dtx, base + e); s += v * v; }
    s = rb::warp_sum(s);
    if (lane == 0) rstd[pair] = 1.f / sqrtf(s / (float)gs + eps);
  }
}

// Packed form.  out[t] = n_t + sum_j cw[:, j] * n_(t - taps + 1 + j), n = grouped RMSNorm(x) * w; sources before the start of
// the sequence (pos[t] < distance) are zero.  taps == 0: out = n.
__global__ void __launch_bounds__(kThreads) sublayer_input_kernel(
    const void* __restrict__ x, int dtx, const void* __restrict__ w, const void* __restrict__ cw, int dta, void* __restrict__ out, int dto,
    const int* __restrict__ pos, float* __restrict__ state, const int* __restrict__ tok_slot, const int* __restrict__ remain,
    int W, int groups, int taps, float eps) {
  extern __shared__ float rstd[];            // [max(taps,1)][groups]
  __shared__ int64_t row_off[kMaxTaps];
  const int64_t t = blockIdx.x;
  const int n_src = taps > 0 ? taps : 1;
  if (threadIdx.x < n_src) {
    const int back = n_src - 1 - threadIdx.x;                         // source row r is `back` tokens before t
    row_off[threadIdx.x] = (back == 0 || (pos != nullptr && pos[t] >= back)) ? t - back : -1;
  }
  __syncthreads();
  group_rstd(x, dtx, row_off, n_src, W, groups, eps, rstd);
  __syncthreads();
  const int gs = W / groups;
  const int slot = (state != nullptr && tok_slot != nullptr) ? tok_slot[t] : -1;
  const int rem = (slot >= 0) ? remain[t] : 1 << 30;
  for (int e = threadIdx.x; e < W; e += blockDim.x) {
    const int g = e / gs;
    const float we = ld_any(w, dta, e);
    const float n_t = ld_any(x, dtx, t * (int64_t)W + e) * rstd[(n_src - 1) * groups + g] * we;
    float h = n_t;
    if (taps > 0) {
      h += ld_any(cw, dta, (int64_t)e * taps + taps - 1) * n_t;
      for (int r = 0; r < taps - 1; ++r) {
        if (row_off[r] < 0) continue;
        const float n_r = ld_any(x, dtx, row_off[r] * (int64_t)W + e) * rstd[r * groups + g] * we;
        h += ld_any(cw, dta, (int64_t)e * taps + r) * n_r;
      }
      if (rem < taps - 1) state[((int64_t)slot * (taps - 1) + (taps - 2 - rem)) * W + e] = n_t;
    }
    st_any(out, dto, t * (int64_t)W + e, h);
  }
}

// One-token form: the earlier inputs are state[slot] ([taps - 1, W], oldest first), shifted by one afterwards.
__global__ void __launch_bounds__(kThreads) sublayer_input_step_kernel(
    const void* __restrict__ x, int dtx, const void* __restrict__ w, const void* __restrict__ cw, int dta, void* __restrict__ out, int dto,
    float* __restrict__ state, const int* __restrict__ slots, int W, int groups, int taps, float eps) {
  extern __shared__ float rstd[];
  __shared__ int64_t row_off[1];
  const int64_t b = blockIdx.x;
  if (threadIdx.x == 0) row_off[0] = b;
  __syncthreads();
  group_rstd(x, dtx, row_off, 1, W, groups, eps, rstd);
  __syncthreads();
  const int gs = W / groups;
  const int64_t slot = slots != nullptr ? slots[b] : b;
  for (int e = threadIdx.x; e < W; e += blockDim.x) {
    const float n_t = ld_any(x, dtx, b * (int64_t)W + e) * rstd[e / gs] * ld_any(w, dta, e);
    float h = n_t;
    if (taps > 0) {
      h += ld_any(cw, dta, (int64_t)e * taps + taps - 1) * n_t;
      float* st = state + slot * (int64_t)(taps - 1) * W + e;
      for (int r = 0; r < taps - 1; ++r) {
        const float v = st[(int64_t)r * W];
        h += ld_any(cw, dta, (int64_t)e * taps + r) * v;
        if (r > 0) st[(int64_t)(r - 1) * W] = v;
      }
      if (taps > 1) st[(int64_t)(taps - 2) * W] = n_t;
    }
    st_any(out, dto, b * (int64_t)W + e, h);
  }
}

// x[t] += grouped RMSNorm(y[t]) * w   (w == nullptr: x[t] += y[t])
__global__ void __launch_bounds__(kThreads) residual_add_norm_kernel(void* __restrict__ x, int dtx, const void* __restrict__ y, int dty,
                                                                     const void* __restrict__ w, int dtw, int W, int groups, float eps) {
  extern __shared__ float rstd[];
  __shared__ int64_t row_off[1];
  const int64_t t = blockIdx.x;
  if (w != nullptr) {
    if (threadIdx.x == 0) row_off[0] = t;
    __syncthreads();
    group_rstd(y, dty, row_off, 1, W, groups, eps, rstd);
    __syncthreads();
  }
  const int gs = W / groups;
  for (int e = threadIdx.x; e < W; e += blockDim.x) {
    float v = ld_any(y, dty, t * (int64_t)W + e);
    if (w != nullptr) v = v * rstd[e / gs] * ld_any(w, dtw, e);
    st_any(x, dtx, t * (int64_t)W + e, ld_any(x, dtx, t * (int64_t)W + e) + v);
  }
}

__global__ void __launch_bounds__(kThreads) clamped_glu_kernel(const void* __restrict__ gu, void* __restrict__ out, int dt, int64_t rows, int F,
                                                               float limit, float alpha) {
  const int64_t total = rows * F;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / F;
    const int c = (int)(i % F);
    const float g = fminf(ld_any(gu, dt, r * 2 * F + c), limit);
    const float u = fminf(fmaxf(ld_any(gu, dt, r * 2 * F + F + c), -limit), limit);
    st_any(out, dt, i, g / (1.f + expf(-alpha * g)) * (u + 1.f));
  }
}

__global__ void __launch_bounds__(kThreads) softcap_kernel(const void* __restrict__ x, int dt, float* __restrict__ out, int64_t n, float cap) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    out[i] = cap * tanhf(ld_any(x, dt, i) / cap);
}

inline int ew_grid(int64_t n) { return (int)std::min<int64_t>(RB_CEIL_DIV(n, (int64_t)kThreads), (int64_t)rb::kNumSMs * 16); }

}  // namespace

extern "C" {

int rb_sublayer_input(const void* x, int dtx, const void* w, const void* cw, int dta, void* out, int dto, const int* pos, float* state,
                      const int* tok_slot, const int* remain, int64_t rows, int W, int groups, int taps, float eps, cudaStream_t s) {
  if (rows == 0) return 0;
  if (groups <= 0 || W % groups != 0 || taps > kMaxTaps || (taps > 1 && pos == nullptr)) return 1;
  const size_t smem = (size_t)(taps > 0 ? taps : 1) * groups * sizeof(float);
  if (smem > 48 * 1024) return 1;
  sublayer_input_kernel<<<(unsigned)rows, kThreads, smem, s>>>(x, dtx, w, cw, dta, out, dto, pos, state, tok_slot, remain, W, groups, taps, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int rb_sublayer_input_step(const void* x, int dtx, const void* w, const void* cw, int dta, void* out, int dto, float* state,
                           const int* slots, int64_t rows, int W, int groups, int taps, float eps, cudaStream_t s) {
  if (rows == 0) return 0;
  if (groups <= 0 || W % groups != 0 || taps > kMaxTaps || (taps > 1 && state == nullptr)) return 1;
  const size_t smem = (size_t)groups * sizeof(float);
  if (smem > 48 * 1024) return 1;
  sublayer_input_step_kernel<<<(unsigned)rows, kThreads, smem, s>>>(x, dtx, w, cw, dta, out, dto, state, slots, W, groups, taps, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int rb_residual_add_norm(void* x, int dtx, const void* y, int dty, const void* w, int dtw, int64_t rows, int W, int groups, float eps,
                         cudaStream_t s) {
  if (rows == 0) return 0;
  if (groups <= 0 || W % groups != 0) return 1;
  const size_t smem = (size_t)groups * sizeof(float);
  if (smem > 48 * 1024) return 1;
  residual_add_norm_kernel<<<(unsigned)rows, kThreads, smem, s>>>(x, dtx, y, dty, w, dtw, W, groups, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int rb_clamped_glu(const void* gu, void* out, int dt, int64_t rows, int F, float limit, float alpha, cudaStream_t s) {
  if (rows * F == 0) return 0;
  clamped_glu_kernel<<<ew_grid(rows * F), kThreads, 0, s>>>(gu, out, dt, rows, F, limit, alpha);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int rb_softcap(const void* x, int dt, float* out, int64_t n, float cap, cudaStream_t s) {
  if (n == 0) return 0;
  softcap_kernel<<<ew_grid(n), kThreads, 0, s>>>(x, dt, out, n, cap);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
