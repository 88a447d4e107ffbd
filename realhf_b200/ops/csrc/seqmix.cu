// Row-wise mechanisms of heterogeneous stacks: grouped RMSNorm fused with a short causal convolution over time (packed and
// one-token forms, the latter with its per-sequence state), residual add fused with a grouped RMSNorm of the branch output,
// the clamped gated-linear-unit activation and the soft cap on logits.
//
// All arithmetic is fp32 whatever the storage types (a type code per tensor: the residual stream is fp32 when the model keeps an
// fp32 residual, activations / weights have the model's type).  A CTA owns a few groups of one row; a (row, group) root mean
// square is reduced by ONE warp in a fixed order, so results do not depend on the batch a row is in.  Rows whose group size is a
// multiple of 4 take 16-byte / 8-byte accesses.  Compiled without fast-math.
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

// 4 consecutive elements starting at index i (i % 4 == 0, base pointers 16-byte aligned: checked by the launchers)
RB_DEVICE float4 ld4_any(const void* p, int dt, int64_t i) {
  if (dt == 0) return *reinterpret_cast<const float4*>(static_cast<const float*>(p) + i);
  const uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(p) + i);
  if (dt == 1) {
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
  }
  const __half2 a = *reinterpret_cast<const __half2*>(&raw.x), b = *reinterpret_cast<const __half2*>(&raw.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
RB_DEVICE void st4_any(void* p, int dt, int64_t i, float4 v) {
  if (dt == 0) { *reinterpret_cast<float4*>(static_cast<float*>(p) + i) = v; return; }
  uint2 raw;
  if (dt == 1) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    raw.x = *reinterpret_cast<const uint32_t*>(&a); raw.y = *reinterpret_cast<const uint32_t*>(&b);
  } else {
    const __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
    raw.x = *reinterpret_cast<const uint32_t*>(&a); raw.y = *reinterpret_cast<const uint32_t*>(&b);
  }
  *reinterpret_cast<uint2*>(static_cast<uint16_t*>(p) + i) = raw;
}

// A CTA owns `gpb` consecutive groups of one row (grid = rows x ceil(groups / gpb)): rows of a decode batch are few, so the
// groups supply the parallelism; in a packed prefill a CTA takes several groups.  rstd[r * gpb + g] of the CTA's groups for
// `n_rows` source rows (row r at x + row_off[r] * W, skipped when row_off[r] < 0): one warp per (row, group), fixed order.
template <bool kVec>
RB_DEVICE void group_rstd(const void* x, int dtx, const int64_t* row_off, int n_rows, int W, int gs, int g0, int ng, float eps, float* rstd) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  for (int pair = warp; pair < n_rows * ng; pair += nwarp) {
    const int r = pair / ng, g = pair % ng;
    if (row_off[r] < 0) continue;
    const int64_t base = row_off[r] * (int64_t)W + (int64_t)(g0 + g) * gs;
    float s = 0.f;
    if constexpr (kVec) {
      for (int e = lane * 4; e < gs; e += 128) { const float4 v = ld4_any(x, dtx, base + e); s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w; }
    } else {
      for (int e = lane; e < gs; e += 32) { const float v = ld_any(x, dtx, base + e); s += v * v; }
    }
    s = rb::warp_sum(s);
    if (lane == 0) rstd[r * ng + g] = 1.f / sqrtf(s / (float)gs + eps);
  }
}

RB_DEVICE float4 mul4(float4 a, float4 b) { return make_float4(a.x * b.x, a.y * b.y, a.z * b.z, a.w * b.w); }
RB_DEVICE float4 scl4(float4 a, float s) { return make_float4(a.x * s, a.y * s, a.z * s, a.w * s); }
RB_DEVICE float4 fma4(float4 a, float4 b, float4 c) { return make_float4(fmaf(a.x, b.x, c.x), fmaf(a.y, b.y, c.y), fmaf(a.z, b.z, c.z), fmaf(a.w, b.w, c.w)); }

// The convolution weights arrive tap-major, [taps, W] (the op layer keeps a transposed copy of the model's [W, taps] tensor), so
// the weights of consecutive channels for one tap are one vector load.

// Packed form.  out[t] = n_t + sum_j cw[:, j] * n_(t - taps + 1 + j), n = grouped RMSNorm(x) * w; sources before the start of
// the sequence (pos[t] < distance) are zero.  taps == 0: out = n.
template <bool kVec>
__global__ void __launch_bounds__(kThreads) sublayer_input_kernel(
    const void* __restrict__ x, int dtx, const void* __restrict__ w, const void* __restrict__ cw, int dta, void* __restrict__ out, int dto,
    const int* __restrict__ pos, float* __restrict__ state, const int* __restrict__ tok_slot, const int* __restrict__ remain,
    int W, int groups, int gpb, int taps, float eps) {
  extern __shared__ float rstd[];            // [max(taps,1)][ng]
  __shared__ int64_t row_off[kMaxTaps];
  const int64_t t = blockIdx.x;
  const int g0 = blockIdx.y * gpb, ng = min(gpb, groups - g0), gs = W / groups;
  const int n_src = taps > 0 ? taps : 1;
  if (threadIdx.x < n_src) {
    const int back = n_src - 1 - threadIdx.x;                         // source row r is `back` tokens before t
    row_off[threadIdx.x] = (back == 0 || (pos != nullptr && pos[t] >= back)) ? t - back : -1;
  }
  __syncthreads();
  group_rstd<kVec>(x, dtx, row_off, n_src, W, gs, g0, ng, eps, rstd);
  __syncthreads();
  const int slot = (state != nullptr && tok_slot != nullptr) ? tok_slot[t] : -1;
  const int rem = (slot >= 0) ? remain[t] : 1 << 30;
  const int e0 = g0 * gs, e1 = e0 + ng * gs;
  if constexpr (kVec) {
    for (int e = e0 + threadIdx.x * 4; e < e1; e += blockDim.x * 4) {
      const int g = (e - e0) / gs;
      const float4 we = ld4_any(w, dta, e);
      const float4 n_t = mul4(scl4(ld4_any(x, dtx, t * (int64_t)W + e), rstd[(n_src - 1) * ng + g]), we);
      float4 h = n_t;
      if (taps > 0) {
        h = fma4(ld4_any(cw, dta, (int64_t)(taps - 1) * W + e), n_t, h);
        for (int r = 0; r < taps - 1; ++r) {
          if (row_off[r] < 0) continue;
          const float4 n_r = mul4(scl4(ld4_any(x, dtx, row_off[r] * (int64_t)W + e), rstd[r * ng + g]), we);
          h = fma4(ld4_any(cw, dta, (int64_t)r * W + e), n_r, h);
        }
        if (rem < taps - 1) *reinterpret_cast<float4*>(state + ((int64_t)slot * (taps - 1) + (taps - 2 - rem)) * W + e) = n_t;
      }
      st4_any(out, dto, t * (int64_t)W + e, h);
    }
  } else {
    for (int e = e0 + threadIdx.x; e < e1; e += blockDim.x) {
      const int g = (e - e0) / gs;
      const float we = ld_any(w, dta, e);
      const float n_t = ld_any(x, dtx, t * (int64_t)W + e) * rstd[(n_src - 1) * ng + g] * we;
      float h = n_t;
      if (taps > 0) {
        h += ld_any(cw, dta, (int64_t)(taps - 1) * W + e) * n_t;
        for (int r = 0; r < taps - 1; ++r) {
          if (row_off[r] < 0) continue;
          const float n_r = ld_any(x, dtx, row_off[r] * (int64_t)W + e) * rstd[r * ng + g] * we;
          h += ld_any(cw, dta, (int64_t)r * W + e) * n_r;
        }
        if (rem < taps - 1) state[((int64_t)slot * (taps - 1) + (taps - 2 - rem)) * W + e] = n_t;
      }
      st_any(out, dto, t * (int64_t)W + e, h);
    }
  }
}

// Packed form, token-tiled: a CTA owns kTT consecutive packed tokens x a chunk of groups.  The tile's rows and the taps - 1
// rows before it are staged once in shared memory (raw fp32), every (row, group) root mean square is reduced from there by one
// warp, and each thread then produces its 4 channels for all tokens of the tile with the norm and tap weights in registers: a
// row of x is read once per tile instead of once per tap.  Same arithmetic, in the same order per element, as the row kernel.
constexpr int kTT = 8;

__global__ void __launch_bounds__(kThreads) sublayer_input_tiled_kernel(
    const void* __restrict__ x, int dtx, const void* __restrict__ w, const void* __restrict__ cw, int dta, void* __restrict__ out, int dto,
    const int* __restrict__ pos, float* __restrict__ state, const int* __restrict__ tok_slot, const int* __restrict__ remain,
    int64_t n_tok, int W, int groups, int gpb, int taps, float eps) {
  extern __shared__ float sm[];
  const int g0 = blockIdx.y * gpb, ng = min(gpb, groups - g0), gs = W / groups;
  const int E = ng * gs, e0 = g0 * gs;
  const int halo = taps - 1, n_rows = kTT + halo;
  float* raw = sm;                           // [n_rows][E]
  float* rstd = sm + (size_t)n_rows * gpb * gs;   // [n_rows][ng]
  const int64_t t0 = (int64_t)blockIdx.x * kTT;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  for (int q = threadIdx.x; q < n_rows * (E / 4); q += blockDim.x) {
    const int r = q / (E / 4), c = (q - r * (E / 4)) * 4;
    const int64_t t = t0 - halo + r;
    const float4 v = (t >= 0 && t < n_tok) ? ld4_any(x, dtx, t * (int64_t)W + e0 + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    *reinterpret_cast<float4*>(raw + (size_t)r * E + c) = v;
  }
  __syncthreads();
  for (int pair = warp; pair < n_rows * ng; pair += nwarp) {
    const int r = pair / ng, g = pair - r * ng;
    const float* src = raw + (size_t)r * E + g * gs;
    float s = 0.f;
    for (int e = lane * 4; e < gs; e += 128) { const float4 v = *reinterpret_cast<const float4*>(src + e); s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w; }
    s = rb::warp_sum(s);
    if (lane == 0) rstd[pair] = 1.f / sqrtf(s / (float)gs + eps);
  }
  __syncthreads();
  for (int c = threadIdx.x * 4; c < E; c += blockDim.x * 4) {
    const int g = c / gs, e = e0 + c;
    const float4 we = ld4_any(w, dta, e);
    float4 cwj[kMaxTaps];
    for (int j = 0; j < taps; ++j) cwj[j] = ld4_any(cw, dta, (int64_t)j * W + e);
    for (int i = 0; i < kTT; ++i) {
      const int64_t t = t0 + i;
      if (t >= n_tok) break;
      const int row = i + halo, p = pos[t];
      const float4 n_t = mul4(scl4(*reinterpret_cast<const float4*>(raw + (size_t)row * E + c), rstd[row * ng + g]), we);
      float4 h = fma4(cwj[taps - 1], n_t, n_t);
      for (int r = 0; r < taps - 1; ++r) {
        const int back = taps - 1 - r;
        if (p < back) continue;
        const float4 n_r = mul4(scl4(*reinterpret_cast<const float4*>(raw + (size_t)(row - back) * E + c), rstd[(row - back) * ng + g]), we);
        h = fma4(cwj[r], n_r, h);
      }
      if (state != nullptr) {
        const int slot = tok_slot[t], rem = remain[t];
        if (slot >= 0 && rem < taps - 1) *reinterpret_cast<float4*>(state + ((int64_t)slot * (taps - 1) + (taps - 2 - rem)) * W + e) = n_t;
      }
      st4_any(out, dto, t * (int64_t)W + e, h);
    }
  }
}

// One-token form: the earlier inputs are state[slot] ([taps - 1, W], oldest first), shifted by one afterwards.
template <bool kVec>
__global__ void __launch_bounds__(kThreads) sublayer_input_step_kernel(
    const void* __restrict__ x, int dtx, const void* __restrict__ w, const void* __restrict__ cw, int dta, void* __restrict__ out, int dto,
    float* __restrict__ state, const int* __restrict__ slots, int W, int groups, int gpb, int taps, float eps) {
  extern __shared__ float rstd[];
  __shared__ int64_t row_off[1];
  const int64_t b = blockIdx.x;
  const int g0 = blockIdx.y * gpb, ng = min(gpb, groups - g0), gs = W / groups;
  if (threadIdx.x == 0) row_off[0] = b;
  __syncthreads();
  group_rstd<kVec>(x, dtx, row_off, 1, W, gs, g0, ng, eps, rstd);
  __syncthreads();
  const int64_t slot = slots != nullptr ? slots[b] : b;
  const int e0 = g0 * gs, e1 = e0 + ng * gs;
  if constexpr (kVec) {
    for (int e = e0 + threadIdx.x * 4; e < e1; e += blockDim.x * 4) {
      const float4 n_t = mul4(scl4(ld4_any(x, dtx, b * (int64_t)W + e), rstd[(e - e0) / gs]), ld4_any(w, dta, e));
      float4 h = n_t;
      if (taps > 0) {
        h = fma4(ld4_any(cw, dta, (int64_t)(taps - 1) * W + e), n_t, h);
        float* st = state + slot * (int64_t)(taps - 1) * W + e;
        for (int r = 0; r < taps - 1; ++r) {
          const float4 v = *reinterpret_cast<const float4*>(st + (int64_t)r * W);
          h = fma4(ld4_any(cw, dta, (int64_t)r * W + e), v, h);
          if (r > 0) *reinterpret_cast<float4*>(st + (int64_t)(r - 1) * W) = v;
        }
        if (taps > 1) *reinterpret_cast<float4*>(st + (int64_t)(taps - 2) * W) = n_t;
      }
      st4_any(out, dto, b * (int64_t)W + e, h);
    }
  } else {
    for (int e = e0 + threadIdx.x; e < e1; e += blockDim.x) {
      const float n_t = ld_any(x, dtx, b * (int64_t)W + e) * rstd[(e - e0) / gs] * ld_any(w, dta, e);
      float h = n_t;
      if (taps > 0) {
        h += ld_any(cw, dta, (int64_t)(taps - 1) * W + e) * n_t;
        float* st = state + slot * (int64_t)(taps - 1) * W + e;
        for (int r = 0; r < taps - 1; ++r) {
          const float v = st[(int64_t)r * W];
          h += ld_any(cw, dta, (int64_t)r * W + e) * v;
          if (r > 0) st[(int64_t)(r - 1) * W] = v;
        }
        if (taps > 1) st[(int64_t)(taps - 2) * W] = n_t;
      }
      st_any(out, dto, b * (int64_t)W + e, h);
    }
  }
}

// x[t] += grouped RMSNorm(y[t]) * w   (w == nullptr: x[t] += y[t])
template <bool kVec>
__global__ void __launch_bounds__(kThreads) residual_add_norm_kernel(void* __restrict__ x, int dtx, const void* __restrict__ y, int dty,
                                                                     const void* __restrict__ w, int dtw, int W, int groups, int gpb, float eps) {
  extern __shared__ float rstd[];
  __shared__ int64_t row_off[1];
  const int64_t t = blockIdx.x;
  const int g0 = blockIdx.y * gpb, ng = min(gpb, groups - g0), gs = W / groups;
  if (w != nullptr) {
    if (threadIdx.x == 0) row_off[0] = t;
    __syncthreads();
    group_rstd<kVec>(y, dty, row_off, 1, W, gs, g0, ng, eps, rstd);
    __syncthreads();
  }
  const int e0 = g0 * gs, e1 = e0 + ng * gs;
  if constexpr (kVec) {
    for (int e = e0 + threadIdx.x * 4; e < e1; e += blockDim.x * 4) {
      float4 v = ld4_any(y, dty, t * (int64_t)W + e);
      if (w != nullptr) v = mul4(scl4(v, rstd[(e - e0) / gs]), ld4_any(w, dtw, e));
      const float4 xv = ld4_any(x, dtx, t * (int64_t)W + e);
      st4_any(x, dtx, t * (int64_t)W + e, make_float4(xv.x + v.x, xv.y + v.y, xv.z + v.z, xv.w + v.w));
    }
  } else {
    for (int e = e0 + threadIdx.x; e < e1; e += blockDim.x) {
      float v = ld_any(y, dty, t * (int64_t)W + e);
      if (w != nullptr) v = v * rstd[(e - e0) / gs] * ld_any(w, dtw, e);
      st_any(x, dtx, t * (int64_t)W + e, ld_any(x, dtx, t * (int64_t)W + e) + v);
    }
  }
}

// groups per CTA: about 2048 elements per CTA when rows are plenty, one group per CTA when rows are few (decode)
inline int groups_per_block(int64_t rows, int W, int groups) {
  const int gs = W / groups;
  int gpb = std::max(1, std::min(groups, 2048 / std::max(gs, 1)));
  while (gpb > 1 && rows * RB_CEIL_DIV(groups, gpb) < 4 * rb::kNumSMs) gpb = (gpb + 1) / 2;
  return gpb;
}
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

RB_DEVICE float clamped_glu_1(float g, float u, float limit, float alpha) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.f + expf(-alpha * g)) * (u + 1.f);
}

template <bool kVec>
__global__ void __launch_bounds__(kThreads) clamped_glu_kernel(const void* __restrict__ gu, void* __restrict__ out, int dt, int64_t rows, int F,
                                                               float limit, float alpha) {
  if constexpr (kVec) {
    const int F4 = F / 4;
    const int64_t total = rows * F4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
      const int64_t r = i / F4;
      const int c = (int)(i % F4) * 4;
      const float4 g = ld4_any(gu, dt, r * 2 * F + c), u = ld4_any(gu, dt, r * 2 * F + F + c);
      st4_any(out, dt, r * F + c, make_float4(clamped_glu_1(g.x, u.x, limit, alpha), clamped_glu_1(g.y, u.y, limit, alpha),
                                               clamped_glu_1(g.z, u.z, limit, alpha), clamped_glu_1(g.w, u.w, limit, alpha)));
    }
  } else {
    const int64_t total = rows * F;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
      const int64_t r = i / F;
      const int c = (int)(i % F);
      st_any(out, dt, i, clamped_glu_1(ld_any(gu, dt, r * 2 * F + c), ld_any(gu, dt, r * 2 * F + F + c), limit, alpha));
    }
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
  const int gpb = groups_per_block(rows, W, groups);
  const size_t smem = (size_t)(taps > 0 ? taps : 1) * gpb * sizeof(float);
  if (smem > 48 * 1024) return 1;
  const bool vec = (W / groups) % 4 == 0 && aligned16(x) && aligned16(w) && aligned16(out) && (state == nullptr || aligned16(state)) &&
                   (cw == nullptr || aligned16(cw));
  if (vec && taps > 1 && rows >= 4 * kTT * rb::kNumSMs) {   // long packed batches: token tiles (each row of x is read once per tile)
    int gt = std::max(1, std::min(groups, 1024 / std::max(W / groups, 1)));
    const size_t smem_t = (size_t)(kTT + taps - 1) * gt * ((size_t)(W / groups) + 1) * sizeof(float);
    if (smem_t <= 100 * 1024) {
      static bool attr_set = false;
      if (!attr_set) {
        if (cudaFuncSetAttribute(sublayer_input_tiled_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024) != cudaSuccess) return 2;
        attr_set = true;
      }
      dim3 grid_t((unsigned)RB_CEIL_DIV(rows, (int64_t)kTT), (unsigned)RB_CEIL_DIV(groups, gt));
      sublayer_input_tiled_kernel<<<grid_t, kThreads, smem_t, s>>>(x, dtx, w, cw, dta, out, dto, pos, state, tok_slot, remain, rows, W, groups,
                                                                   gt, taps, eps);
      return cudaGetLastError() == cudaSuccess ? 0 : 2;
    }
  }
  dim3 grid((unsigned)rows, (unsigned)RB_CEIL_DIV(groups, gpb));
  auto kern = vec ? sublayer_input_kernel<true> : sublayer_input_kernel<false>;
  kern<<<grid, kThreads, smem, s>>>(x, dtx, w, cw, dta, out, dto, pos, state, tok_slot, remain, W, groups, gpb, taps, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int rb_sublayer_input_step(const void* x, int dtx, const void* w, const void* cw, int dta, void* out, int dto, float* state,
                           const int* slots, int64_t rows, int W, int groups, int taps, float eps, cudaStream_t s) {
  if (rows == 0) return 0;
  if (groups <= 0 || W % groups != 0 || taps > kMaxTaps || (taps > 1 && state == nullptr)) return 1;
  const int gpb = groups_per_block(rows, W, groups);
  const size_t smem = (size_t)gpb * sizeof(float);
  if (smem > 48 * 1024) return 1;
  const bool vec = (W / groups) % 4 == 0 && aligned16(x) && aligned16(w) && aligned16(out) && (state == nullptr || aligned16(state)) &&
                   (cw == nullptr || aligned16(cw));
  dim3 grid((unsigned)rows, (unsigned)RB_CEIL_DIV(groups, gpb));
  auto kern = vec ? sublayer_input_step_kernel<true> : sublayer_input_step_kernel<false>;
  kern<<<grid, kThreads, smem, s>>>(x, dtx, w, cw, dta, out, dto, state, slots, W, groups, gpb, taps, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int rb_residual_add_norm(void* x, int dtx, const void* y, int dty, const void* w, int dtw, int64_t rows, int W, int groups, float eps,
                         cudaStream_t s) {
  if (rows == 0) return 0;
  if (groups <= 0 || W % groups != 0) return 1;
  const int gpb = groups_per_block(rows, W, groups);
  const size_t smem = (size_t)gpb * sizeof(float);
  if (smem > 48 * 1024) return 1;
  const bool vec = (W / groups) % 4 == 0 && aligned16(x) && aligned16(y) && (w == nullptr || aligned16(w));
  dim3 grid((unsigned)rows, (unsigned)RB_CEIL_DIV(groups, gpb));
  auto kern = vec ? residual_add_norm_kernel<true> : residual_add_norm_kernel<false>;
  kern<<<grid, kThreads, smem, s>>>(x, dtx, y, dty, w, dtw, W, groups, gpb, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int rb_clamped_glu(const void* gu, void* out, int dt, int64_t rows, int F, float limit, float alpha, cudaStream_t s) {
  if (rows * F == 0) return 0;
  if (F % 4 == 0 && aligned16(gu) && aligned16(out))
    clamped_glu_kernel<true><<<ew_grid(rows * F / 4), kThreads, 0, s>>>(gu, out, dt, rows, F, limit, alpha);
  else
    clamped_glu_kernel<false><<<ew_grid(rows * F), kThreads, 0, s>>>(gu, out, dt, rows, F, limit, alpha);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int rb_softcap(const void* x, int dt, float* out, int64_t n, float cap, cudaStream_t s) {
  if (n == 0) return 0;
  softcap_kernel<<<ew_grid(n), kThreads, 0, s>>>(x, dt, out, n, cap);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
