// Gated delta rule (`DeltaRuleConfig`), packed (prefill) and one-token (decode) forms.  Per head, matrix state S [d, dv] in fp32:
//     S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q          (the output is read after the update)
// All arithmetic that enters the recurrence is fp32; exact expf / log1pf (compiled without fast-math).
//
//   delta_prepare    projection output `proj` [T, ld] = [q (G x d) | k (G x d) | v (H x dv) | gate (H x dv) | beta logits (H) | decay
//                    inputs (H) | pad]  ->  u [T, C + 2H] fp32 = [q | k | v | beta | g],  C = 2 G d + H dv:
//                    causal depthwise convolution (taps <= 8, weights [C, taps], tap taps - 1 meets the current token, inputs before a
//                    sequence's first token are zero) + SiLU on the first C channels; q, k <- x / sqrt(sum x^2 + unit_eps) per head, q also times
//                    d^-1/2; beta = sigmoid; g = exp(-exp(A_log) softplus(a + dt_bias)).  Packed form: earlier tokens are the
//                    preceding rows (pos[t] tells how many belong to the sequence), and the last taps - 1 raw inputs of every
//                    sequence go to conv_state [n_slots, taps - 1, C] (oldest first).  Step form (pos == null): earlier inputs
//                    come from conv_state[slot], which is shifted by one.
// Kernels on the decode path are launched with programmatic dependent launch (they signal their successors at once and wait for
// their predecessor before the first global access), like the framework's other decode kernels.
//   delta_rule       the recurrence.  A column of S depends only on its own v column, so columns are independent: a thread group of
//                    LPC lanes owns one column (32 or 64 state rows per lane in registers), a CTA 128 / LPC columns of one
//                    (sequence, head).  q, k, v, beta, g of 8 tokens at a time are staged in shared memory.  Packed form: S starts
//                    at zero and the final S goes to s_state[slot]; step form: S is loaded from and stored to s_state[slot].
//   gated_head_norm  o / sqrt(mean(o^2) + eps) * w * silu(gate) per (token, head) -> model type.
#include "anytype.cuh"

namespace {

using rb::ld_any;
using rb::st_any;

constexpr int kMaxTaps = 8;

// One CTA per (token, unit); a unit is a q or k head, a v head, or the 2H gate scalars (as in the tiled kernel below), so that a
// decode batch of a few rows still spreads over the GPU.
__global__ void __launch_bounds__(128) delta_prepare_kernel(const void* __restrict__ proj, int64_t ld, int dt, const void* __restrict__ conv_w,
                                                            const void* __restrict__ A_log, const void* __restrict__ dt_bias,
                                                            float* __restrict__ u, const int* __restrict__ pos, float* __restrict__ conv_state,
                                                            const int* __restrict__ tok_slot, const int* __restrict__ remain,
                                                            const int* __restrict__ slots, int H, int G, int d, int dv, int taps,
                                                            float unit_eps) {
  extern __shared__ float ys[];               // [channels of the unit] convolved + SiLU
  __shared__ float red[32];
  const int64_t t = blockIdx.x;
  const int unit = blockIdx.y;
  const int nqk = G * d, nv = H * dv, C = 2 * nqk + nv, UW = C + 2 * H;
  rb::pdl_trigger();
  rb::pdl_wait();
  if (unit == 2 * G + H) {
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
      const float b = ld_any(proj, dt, t * ld + C + nv + h);
      u[t * UW + C + h] = 1.f / (1.f + expf(-b));
      const float a = ld_any(proj, dt, t * ld + C + nv + H + h) + ld_any(dt_bias, dt, h);
      const float sp = a > 20.f ? a : log1pf(expf(a));
      u[t * UW + C + H + h] = expf(-expf(ld_any(A_log, dt, h)) * sp);
    }
    return;
  }
  const bool is_qk = unit < 2 * G;
  const int us = is_qk ? d : dv;
  const int c_base = is_qk ? unit * d : 2 * nqk + (unit - 2 * G) * dv;
  const bool step = pos == nullptr;
  const int p = step ? 0 : pos[t];
  int slot = -1;
  if (conv_state != nullptr) slot = step ? (slots ? slots[t] : (int)t) : tok_slot[t];
  const int rem = (!step && conv_state != nullptr) ? remain[t] : 0;
  float* st = (slot >= 0 && taps > 1) ? conv_state + (int64_t)slot * (taps - 1) * C : nullptr;
  float ss = 0.f;
  for (int cl = threadIdx.x; cl < us; cl += blockDim.x) {
    const int c = c_base + cl;
    const float x = ld_any(proj, dt, t * ld + c);
    float hist[kMaxTaps - 1];
    float y = 0.f;
#pragma unroll
    for (int back = kMaxTaps - 1; back >= 1; --back) {       // oldest first, the current token last: the tiled kernel's order
      if (back < taps) {
        float xb;
        if (step) xb = st ? st[(int64_t)(taps - 1 - back) * C + c] : 0.f;
        else xb = back <= p ? ld_any(proj, dt, (t - back) * ld + c) : 0.f;
        hist[back - 1] = xb;
        y = fmaf(xb, ld_any(conv_w, dt, (int64_t)c * taps + taps - 1 - back), y);
      }
    }
    y = fmaf(x, ld_any(conv_w, dt, (int64_t)c * taps + taps - 1), y);
    if (st != nullptr) {
      if (step) {           // shift: row i <- row i + 1, the newest row <- x (this thread owns channel c of the slot)
#pragma unroll
        for (int back = kMaxTaps - 1; back >= 1; --back)
          if (back < taps) st[(int64_t)(taps - 1 - back) * C + c] = back == 1 ? x : hist[back - 2];
      } else if (rem < taps - 1) {
        st[(int64_t)(taps - 2 - rem) * C + c] = x;
      }
    }
    y = y / (1.f + expf(-y));
    ys[cl] = y;
    ss = fmaf(y, y, ss);
  }
  float r = 1.f;
  if (is_qk) {
    ss = rb::block_reduce<false>(ss, red);
    r = 1.f / sqrtf(ss + unit_eps);
    if (unit < G) r *= 1.f / sqrtf((float)d);
  }
  for (int cl = threadIdx.x; cl < us; cl += blockDim.x) u[t * UW + c_base + cl] = ys[cl] * r;   // a thread re-reads its own entries
}

// Packed form for long batches: a CTA owns 16 consecutive tokens x one unit of channels (a q or k head, a v head, or the 2H gate
// scalars).  A thread keeps its channels' taps and a sliding window of the last taps - 1 inputs in registers and walks the tokens,
// so every input is read once (plus a halo of taps - 1 rows per tile) and the weights once per CTA; the per-(token, head) sums of
// squares are reduced per warp into shared memory and applied after one barrier.
constexpr int kPT = 16, kPThreads = 128;   // tokens per tile, threads; CH channels per thread (units of up to CH * 128 channels)

template <int CH>
__global__ void __launch_bounds__(kPThreads) delta_prepare_tiled_kernel(const void* __restrict__ proj, int64_t ld, int dt, const void* __restrict__ conv_w,
                                                                        const void* __restrict__ A_log, const void* __restrict__ dt_bias,
                                                                        float* __restrict__ u, const int* __restrict__ pos,
                                                                        float* __restrict__ conv_state, const int* __restrict__ tok_slot,
                                                                        const int* __restrict__ remain, int64_t T, int H, int G, int d, int dv,
                                                                        int taps, float unit_eps) {
  __shared__ float part[kPThreads / 32][kPT];
  const int nqk = G * d, nv = H * dv, C = 2 * nqk + nv, UW = C + 2 * H;
  const int unit = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t t0 = (int64_t)blockIdx.x * kPT;
  const int nt = (int)min((int64_t)kPT, T - t0);
  if (unit == 2 * G + H) {   // write strength and decay of every head
    for (int idx = tid; idx < nt * H; idx += kPThreads) {
      const int64_t t = t0 + idx / H;
      const int h = idx % H;
      const float b = ld_any(proj, dt, t * ld + C + nv + h);
      u[t * UW + C + h] = 1.f / (1.f + expf(-b));
      const float a = ld_any(proj, dt, t * ld + C + nv + H + h) + ld_any(dt_bias, dt, h);
      const float sp = a > 20.f ? a : log1pf(expf(a));
      u[t * UW + C + H + h] = expf(-expf(ld_any(A_log, dt, h)) * sp);
    }
    return;
  }
  const bool is_qk = unit < 2 * G;
  const int us = is_qk ? d : dv;                       // channels of this unit
  const int c_base = is_qk ? unit * d : 2 * nqk + (unit - 2 * G) * dv;
  // all loads of the tile first (independent, in flight together), then the arithmetic
  int ps[kPT];
#pragma unroll
  for (int tt = 0; tt < kPT; ++tt) ps[tt] = tt < nt ? pos[t0 + tt] : 0;
  float w[CH][kMaxTaps], hist[CH][kMaxTaps - 1], xv[CH][kPT];
  bool okc[CH];
#pragma unroll
  for (int ch = 0; ch < CH; ++ch) {
    okc[ch] = tid + ch * kPThreads < us;
    const int c = c_base + tid + ch * kPThreads;
#pragma unroll
    for (int tt = 0; tt < kPT; ++tt) xv[ch][tt] = (okc[ch] && tt < nt) ? ld_any(proj, dt, (t0 + tt) * ld + c) : 0.f;
#pragma unroll
    for (int back = 0; back < kMaxTaps; ++back)      // w[ch][back]: the tap that meets the input `back` tokens ago
      w[ch][back] = (okc[ch] && back < taps) ? ld_any(conv_w, dt, (int64_t)c * taps + taps - 1 - back) : 0.f;
#pragma unroll
    for (int back = 1; back < kMaxTaps; ++back)
      hist[ch][back - 1] = (okc[ch] && back < taps && t0 - back >= 0) ? ld_any(proj, dt, (t0 - back) * ld + c) : 0.f;
  }
  if (conv_state != nullptr && taps > 1) {
#pragma unroll
    for (int tt = 0; tt < kPT; ++tt) {
      if (tt < nt) {
        const int slot = tok_slot[t0 + tt], rem = remain[t0 + tt];
        if (slot >= 0 && rem < taps - 1) {
#pragma unroll
          for (int ch = 0; ch < CH; ++ch)
            if (okc[ch]) conv_state[((int64_t)slot * (taps - 1) + (taps - 2 - rem)) * C + c_base + tid + ch * kPThreads] = xv[ch][tt];
        }
      }
    }
  }
#pragma unroll
  for (int tt = 0; tt < kPT; ++tt) {
    float ss = 0.f;
    if (tt < nt) {
      const int p = ps[tt];
#pragma unroll
      for (int ch = 0; ch < CH; ++ch) {
        const float x = xv[ch][tt];
        float y = 0.f;
#pragma unroll
        for (int back = kMaxTaps - 1; back >= 1; --back)      // oldest first, the current token last: a fixed order
          if (back < taps && back <= p) y = fmaf(hist[ch][back - 1], w[ch][back], y);
        y = fmaf(x, w[ch][0], y);
#pragma unroll
        for (int back = kMaxTaps - 1; back >= 2; --back) hist[ch][back - 1] = hist[ch][back - 2];
        hist[ch][0] = x;
        y = y / (1.f + expf(-y));
        xv[ch][tt] = y;
        ss = fmaf(y, y, ss);
      }
    }
    if (is_qk) {
      ss = rb::warp_sum(ss);
      if (lane == 0) part[warp][tt] = ss;
    }
  }
  if (is_qk) __syncthreads();
#pragma unroll
  for (int tt = 0; tt < kPT; ++tt) {
    if (tt < nt) {
      float r = 1.f;
      if (is_qk) {
        r = 1.f / sqrtf(part[0][tt] + part[1][tt] + part[2][tt] + part[3][tt] + unit_eps);
        if (unit < G) r *= 1.f / sqrtf((float)d);
      }
#pragma unroll
      for (int ch = 0; ch < CH; ++ch)
        if (okc[ch]) u[(t0 + tt) * UW + c_base + tid + ch * kPThreads] = xv[ch][tt] * r;
    }
  }
}

// ------------------------------------------------------------------------------------------------ recurrence
constexpr int kScanThreads = 128, kTok = 8;   // kEPL (template): state rows per lane, 32 or 64

struct ScanParams {
  const float* u; float* o;
  const int* cu;            // packed form: [n_seqs + 1]; step form: null (sequence b = row b, one token)
  float* s_state;           // [n_slots, H, d, dv] or null
  const int* slots;         // per sequence / row; null = identity (step form) or no state (packed form)
  int H, G, d, dv, step;
};

// Row mapping: lane l of a column's LPC lanes holds the state rows ((e / 4) * LPC + l) * 4 + e % 4, e = 0 .. 31, so that its q / k
// operands are 8 aligned float4 reads of shared memory per token (the lanes of a column read neighbouring float4s, the columns of
// a warp the same ones).  Dot products run on four independent accumulators.
template <int LPC, int kEPL>
__global__ void __launch_bounds__(kScanThreads, kEPL == 32 ? 3 : 2) delta_rule_kernel(ScanParams p) {
  constexpr int NCOL = kScanThreads / LPC;
  extern __shared__ __align__(16) float sm[];
  const int seq = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * NCOL;
  const int g = h / (p.H / p.G), d = p.d, dv = p.dv;
  const int nqk = p.G * d, C = 2 * nqk + p.H * dv, UW = C + 2 * p.H;
  const int tid = threadIdx.x, l = tid % LPC, col = c0 + tid / LPC;
  const bool active = col < dv;
  int t0, t1;
  rb::pdl_trigger();
  rb::pdl_wait();
  if (p.step) { t0 = seq; t1 = seq + 1; } else { t0 = p.cu[seq]; t1 = p.cu[seq + 1]; }
  if (t1 <= t0) return;
  const int slot = p.s_state == nullptr ? -1 : (p.slots ? p.slots[seq] : (p.step ? seq : -1));
  float* S_g = slot >= 0 ? p.s_state + (((int64_t)slot * p.H + h) * d) * dv : nullptr;
  constexpr int dpad = kEPL * LPC;                // rows >= d hold zeros and read zero q / k
  constexpr int kBuf = 2 * kTok * dpad + kTok * NCOL + 2 * kTok;   // floats of one staging buffer: q, k, v, (beta, g)
  constexpr int NQ = kTok * dpad / kScanThreads, NV = (kTok * NCOL + kScanThreads - 1) / kScanThreads;
  auto row_of = [&](int e) { return ((e >> 2) * LPC + l) * 4 + (e & 3); };
  float S[kEPL];
#pragma unroll
  for (int e = 0; e < kEPL; ++e) {
    const int row = row_of(e);
    S[e] = (p.step && S_g && active && row < d) ? S_g[(int64_t)row * dv + col] : 0.f;
  }
  // The inputs of the next 8 tokens are fetched into registers while the current 8 are processed out of shared memory (two
  // staging buffers, one barrier per chunk).
  float rq[NQ], rk[NQ], rv[NV], rb = 0.f;
  auto fetch = [&](int tb) {
    const int nt = min(kTok, t1 - tb);
#pragma unroll
    for (int i = 0; i < NQ; ++i) {
      const int idx = tid + i * kScanThreads, tt = idx / dpad, e = idx % dpad;
      const bool ok = tt < nt && e < d;
      const float* row = p.u + (int64_t)(tb + tt) * UW;
      rq[i] = ok ? row[g * d + e] : 0.f;
      rk[i] = ok ? row[nqk + g * d + e] : 0.f;
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int idx = tid + i * kScanThreads, tt = idx / NCOL, c = c0 + idx % NCOL;
      rv[i] = (idx < kTok * NCOL && tt < nt && c < dv) ? p.u[(int64_t)(tb + tt) * UW + 2 * nqk + h * dv + c] : 0.f;
    }
    rb = tid < nt * 2 ? p.u[(int64_t)(tb + tid / 2) * UW + C + (tid & 1) * p.H + h] : 0.f;
  };
  auto stage = [&](float* buf) {
#pragma unroll
    for (int i = 0; i < NQ; ++i) { buf[tid + i * kScanThreads] = rq[i]; buf[kTok * dpad + tid + i * kScanThreads] = rk[i]; }
#pragma unroll
    for (int i = 0; i < NV; ++i)
      if (tid + i * kScanThreads < kTok * NCOL) buf[2 * kTok * dpad + tid + i * kScanThreads] = rv[i];
    if (tid < 2 * kTok) buf[2 * kTok * dpad + kTok * NCOL + tid] = rb;
  };
  fetch(t0);
  int which = 0;
  for (int tb = t0; tb < t1; tb += kTok, which ^= 1) {
    const int nt = min(kTok, t1 - tb);
    float* buf = sm + which * kBuf;
    stage(buf);
    __syncthreads();
    if (tb + kTok < t1) fetch(tb + kTok);
    const float* qs = buf;
    const float* ks = buf + kTok * dpad;
    const float* vs = ks + kTok * dpad;
    const float* bg = vs + kTok * NCOL;
    for (int tt = 0; tt < nt; ++tt) {
      const float beta = bg[tt * 2], gg = bg[tt * 2 + 1];
      const float4* kq = reinterpret_cast<const float4*>(ks + tt * dpad) + l;
      const float4* qq = reinterpret_cast<const float4*>(qs + tt * dpad) + l;
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
      for (int e4 = 0; e4 < kEPL / 4; ++e4) {
        const float4 kk = kq[e4 * LPC];
        S[e4 * 4] *= gg; S[e4 * 4 + 1] *= gg; S[e4 * 4 + 2] *= gg; S[e4 * 4 + 3] *= gg;
        a0 = fmaf(S[e4 * 4], kk.x, a0); a1 = fmaf(S[e4 * 4 + 1], kk.y, a1);
        a2 = fmaf(S[e4 * 4 + 2], kk.z, a2); a3 = fmaf(S[e4 * 4 + 3], kk.w, a3);
      }
      float acc = (a0 + a1) + (a2 + a3);
#pragma unroll
      for (int off = 1; off < LPC; off <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
      const float w = beta * (vs[tt * NCOL + tid / LPC] - acc);
      a0 = a1 = a2 = a3 = 0.f;
#pragma unroll
      for (int e4 = 0; e4 < kEPL / 4; ++e4) {
        const float4 kk = kq[e4 * LPC], q4 = qq[e4 * LPC];
        S[e4 * 4] = fmaf(kk.x, w, S[e4 * 4]); S[e4 * 4 + 1] = fmaf(kk.y, w, S[e4 * 4 + 1]);
        S[e4 * 4 + 2] = fmaf(kk.z, w, S[e4 * 4 + 2]); S[e4 * 4 + 3] = fmaf(kk.w, w, S[e4 * 4 + 3]);
        a0 = fmaf(S[e4 * 4], q4.x, a0); a1 = fmaf(S[e4 * 4 + 1], q4.y, a1);
        a2 = fmaf(S[e4 * 4 + 2], q4.z, a2); a3 = fmaf(S[e4 * 4 + 3], q4.w, a3);
      }
      float ov = (a0 + a1) + (a2 + a3);
#pragma unroll
      for (int off = 1; off < LPC; off <<= 1) ov += __shfl_xor_sync(0xffffffffu, ov, off);
      if (active && l == 0) p.o[((int64_t)(tb + tt) * p.H + h) * dv + col] = ov;
    }
  }
  if (S_g && active) {
#pragma unroll
    for (int e = 0; e < kEPL; ++e) {
      const int row = row_of(e);
      if (row < d) S_g[(int64_t)row * dv + col] = S[e];
    }
  }
}

// one warp per (token, head)
__global__ void __launch_bounds__(128) gated_head_norm_kernel(const float* __restrict__ o, const void* __restrict__ w, int dtw,
                                                              const void* __restrict__ gate, int64_t ldg, int dtg, void* __restrict__ out, int dto,
                                                              int64_t rows, int H, int dv, float eps) {
  const int64_t r = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  rb::pdl_trigger();
  rb::pdl_wait();
  if (r >= rows) return;
  const int lane = threadIdx.x & 31;
  const int64_t t = r / H;
  const int h = (int)(r % H);
  const float* x = o + r * dv;
  float ss = 0.f;
  for (int c = lane; c < dv; c += 32) ss += x[c] * x[c];
  ss = rb::warp_sum(ss);
  const float rs = 1.f / sqrtf(ss / (float)dv + eps);
  for (int c = lane; c < dv; c += 32) {
    const float gt = ld_any(gate, dtg, t * ldg + h * dv + c);
    st_any(out, dto, r * dv + c, x[c] * rs * ld_any(w, dtw, c) * (gt / (1.f + expf(-gt))));
  }
}

}  // namespace

extern "C" int rb_delta_prepare(const void* proj, int64_t ld, int dt, const void* conv_w, const void* A_log, const void* dt_bias, float* u,
                                const int* pos, float* conv_state, const int* tok_slot, const int* remain, const int* slots, int64_t T, int H, int G,
                                int d, int dv, int taps, float unit_eps, cudaStream_t s) {
  if (T == 0) return 0;
  if (taps < 1 || taps > kMaxTaps) return -1;
  const int C = 2 * G * d + H * dv;
  if (pos != nullptr && T >= 64 && d <= 2 * kPThreads && dv <= 2 * kPThreads) {
    dim3 grid((unsigned)((T + kPT - 1) / kPT), 2 * G + H + 1);
    if (d <= kPThreads && dv <= kPThreads)
      delta_prepare_tiled_kernel<1><<<grid, kPThreads, 0, s>>>(proj, ld, dt, conv_w, A_log, dt_bias, u, pos, conv_state, tok_slot, remain, T, H, G, d,
                                                               dv, taps, unit_eps);
    else
      delta_prepare_tiled_kernel<2><<<grid, kPThreads, 0, s>>>(proj, ld, dt, conv_w, A_log, dt_bias, u, pos, conv_state, tok_slot, remain, T, H, G, d,
                                                               dv, taps, unit_eps);
    return 0;
  }
  const size_t smem = sizeof(float) * (size_t)(d > dv ? d : dv);
  if (smem > 48 * 1024) return -2;
  if (rb::launch_pdl(delta_prepare_kernel, dim3((unsigned)T, 2 * G + H + 1), dim3(128), smem, s, proj, ld, dt, conv_w, A_log, dt_bias, u, pos,
                     conv_state, tok_slot, remain, slots, H, G, d, dv, taps, unit_eps) != cudaSuccess)
    return -3;
  return 0;
}

extern "C" int rb_delta_rule(const float* u, float* o, const int* cu, float* s_state, const int* slots, int n_seqs, int H, int G, int d, int dv,
                             int step, cudaStream_t s) {
  if (n_seqs == 0) return 0;
  if (d > 512 || H % G) return -1;
  // (lanes per column, state rows per lane): 64 rows per lane from head size 128 up halves the shuffle rounds and the shared
  // reads per FMA at two CTAs per SM
  const int lpc = d <= 32 ? 1 : d <= 64 ? 2 : d <= 128 ? 2 : d <= 256 ? 4 : 8;
  const int epl = d <= 64 ? 32 : 64;
  const int ncol = kScanThreads / lpc;
  ScanParams p{u, o, cu, s_state, slots, H, G, d, dv, step};
  const size_t smem = 2 * sizeof(float) * ((size_t)2 * kTok * epl * lpc + (size_t)kTok * ncol + 2 * kTok);   // two staging buffers
  dim3 grid(n_seqs, H, RB_CEIL_DIV(dv, ncol));
  cudaError_t e;
  if (epl == 32) {
    if (lpc == 1) e = rb::launch_pdl(delta_rule_kernel<1, 32>, grid, dim3(kScanThreads), smem, s, p);
    else e = rb::launch_pdl(delta_rule_kernel<2, 32>, grid, dim3(kScanThreads), smem, s, p);
  } else {
    if (lpc == 2) e = rb::launch_pdl(delta_rule_kernel<2, 64>, grid, dim3(kScanThreads), smem, s, p);
    else if (lpc == 4) e = rb::launch_pdl(delta_rule_kernel<4, 64>, grid, dim3(kScanThreads), smem, s, p);
    else {
      if (smem > 48 * 1024) cudaFuncSetAttribute(delta_rule_kernel<8, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      e = rb::launch_pdl(delta_rule_kernel<8, 64>, grid, dim3(kScanThreads), smem, s, p);
    }
  }
  return e == cudaSuccess ? 0 : -3;
}

extern "C" int rb_gated_head_norm(const float* o, const void* w, int dtw, const void* gate, int64_t ldg, int dtg, void* out, int dto, int64_t T, int H,
                                  int dv, float eps, cudaStream_t s) {
  const int64_t rows = T * H;
  if (rows == 0) return 0;
  return rb::launch_pdl(gated_head_norm_kernel, dim3((unsigned)((rows + 3) / 4)), dim3(128), 0, s, o, w, dtw, gate, ldg, dtg, out, dto, rows, H, dv,
                        eps) == cudaSuccess ? 0 : -3;
}
