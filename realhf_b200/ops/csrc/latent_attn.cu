// Latent attention: keys and values are up-projections of one cached low-rank latent per token; no positional rotation; an
// optional sliding window (a query at position i sees positions (i - window, i]).
//
//   latent_norm_store        packed prefill: c = RMSNorm(latent part of the fused q|latent projection) * w, written packed
//                            [T, rank] (input of the key/value up-projection GEMM) and into the ring cache of its sequence
//   latent_window_attention  packed prefill over the up-projected keys / values: 16 queries x 1 head per CTA, key tiles staged
//                            in shared memory, online softmax
//   latent_decode_attention  one token per row, keys / values never formed: the query is multiplied into the latent space
//                            (q W_uk), scores and the weighted sum run over the cached latents, W_uv is applied to the result;
//                            a block that owns its latent also normalises and appends the new row
//
// Scores, softmax and all accumulations are fp32; storage is T (bf16 / fp16 / fp32).  Compiled without fast-math.
// The cache of a slot is a ring of R rows: position p lives in row p % R.
#include "common.cuh"

namespace {

// ------------------------------------------------------------------------------------------------ latent_norm_store
template <typename T>
__global__ void __launch_bounds__(128) latent_norm_store_kernel(const T* __restrict__ qc, int64_t ldq, int n_q, const T* __restrict__ w,
                                                                T* __restrict__ c_out, T* __restrict__ cache, const int* __restrict__ tok_slot,
                                                                const int* __restrict__ pos, const int* __restrict__ remain, int64_t n_tok,
                                                                int rank, int R, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= n_tok) return;
  const T* src = qc + t * ldq + n_q;
  float s = 0.f;
  for (int r = lane; r < rank; r += 32) { const float v = rb::to_f(src[r]); s += v * v; }
  s = rb::warp_sum(s);
  const float rstd = 1.f / sqrtf(s / (float)rank + eps);
  // only the last R tokens of a sequence go to its ring: earlier ones would land in rows that later positions own
  const int slot = (cache != nullptr && tok_slot != nullptr && remain[t] < R) ? tok_slot[t] : -1;
  T* dst = slot >= 0 ? cache + ((int64_t)slot * R + (pos[t] % R)) * rank : nullptr;
  for (int r = lane; r < rank; r += 32) {
    const T v = rb::from_f<T>(rb::to_f(src[r]) * rstd * rb::to_f(w[r]));
    c_out[t * rank + r] = v;
    if (dst != nullptr) dst[r] = v;
  }
}

// ------------------------------------------------------------------------------------------------ prefill
constexpr int kBQ = 16;    // queries per CTA
constexpr int kBK = 32;    // keys per shared-memory tile
constexpr int kPT = 128;   // threads: 8 per query

// Thread (i = tid / 8, c = tid % 8) owns query i's scores of keys c, c + 8, c + 16, c + 24 of a tile and its output columns
// c, c + 8, ...  NACC = ceil(vd / 8) accumulators per thread.
template <typename T, int NACC>
__global__ void __launch_bounds__(kPT) latent_window_attention_kernel(const T* __restrict__ q, int64_t ldq, const T* __restrict__ kv, int64_t ldkv,
                                                                      const int* __restrict__ pos, T* __restrict__ out, int64_t n_tok, int H,
                                                                      int qk, int vd, float scale, int window) {
  extern __shared__ float sm[];
  float* qs = sm;                          // [kBQ][qk]
  float* ks = qs + kBQ * qk;               // [kBK][qk + 1]
  float* vs = ks + kBK * (qk + 1);         // [kBK][vd]
  float* ps = vs + kBK * vd;               // [kBQ][kBK]
  __shared__ int64_t lo_s[kBQ];
  const int tid = threadIdx.x, i = tid >> 3, c = tid & 7;
  const int h = blockIdx.y;
  const int64_t t0 = (int64_t)blockIdx.x * kBQ;
  const int nq_valid = (int)min((int64_t)kBQ, n_tok - t0);
  if (tid < kBQ) {
    int64_t lo = INT64_MAX;
    if (tid < nq_valid) {
      const int p = pos[t0 + tid];
      const int reach = (window > 0 && window - 1 < p) ? window - 1 : p;
      lo = t0 + tid - reach;
    }
    lo_s[tid] = lo;
  }
  for (int e = tid; e < kBQ * qk; e += kPT) {
    const int r = e / qk, d = e % qk;
    qs[e] = r < nq_valid ? rb::to_f(q[(t0 + r) * ldq + (int64_t)h * qk + d]) : 0.f;
  }
  __syncthreads();
  int64_t tile_lo = INT64_MAX;
  for (int r = 0; r < nq_valid; ++r) tile_lo = min(tile_lo, lo_s[r]);
  const int64_t tile_hi = t0 + nq_valid - 1;
  const bool q_ok = i < nq_valid;
  const int64_t my_t = t0 + i, my_lo = q_ok ? lo_s[i] : INT64_MAX;
  float m = -INFINITY, l = 0.f, acc[NACC];
#pragma unroll
  for (int a = 0; a < NACC; ++a) acc[a] = 0.f;
  const int64_t k_off = (int64_t)h * qk, v_off = (int64_t)H * qk + (int64_t)h * vd;
  for (int64_t kb = tile_lo; kb <= tile_hi; kb += kBK) {
    const int nk = (int)min((int64_t)kBK, tile_hi - kb + 1);
    for (int e = tid; e < kBK * qk; e += kPT) {
      const int r = e / qk, d = e % qk;
      ks[r * (qk + 1) + d] = r < nk ? rb::to_f(kv[(kb + r) * ldkv + k_off + d]) : 0.f;
    }
    for (int e = tid; e < kBK * vd; e += kPT) {
      const int r = e / vd, d = e % vd;
      vs[e] = r < nk ? rb::to_f(kv[(kb + r) * ldkv + v_off + d]) : 0.f;
    }
    __syncthreads();
    float sc[kBK / 8];
    float cmax = -INFINITY;
#pragma unroll
    for (int jj = 0; jj < kBK / 8; ++jj) {
      const int j = c + 8 * jj;
      const int64_t key = kb + j;
      float s = -INFINITY;
      if (q_ok && j < nk && key >= my_lo && key <= my_t) {
        float d_ = 0.f;
        const float* qr = qs + i * qk;
        const float* kr = ks + j * (qk + 1);
        for (int d = 0; d < qk; ++d) d_ = fmaf(qr[d], kr[d], d_);
        s = d_ * scale;
      }
      sc[jj] = s;
      cmax = fmaxf(cmax, s);
    }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) cmax = fmaxf(cmax, __shfl_xor_sync(0xffffffffu, cmax, o));
    const float m_new = fmaxf(m, cmax);
    float corr = 1.f, psum = 0.f;
    if (m_new == -INFINITY) {                      // no visible key so far: nothing to add
#pragma unroll
      for (int jj = 0; jj < kBK / 8; ++jj) ps[i * kBK + c + 8 * jj] = 0.f;
    } else {
      corr = expf(m - m_new);                      // m = -inf: 0
#pragma unroll
      for (int jj = 0; jj < kBK / 8; ++jj) {
        const float p = expf(sc[jj] - m_new);      // masked: exp(-inf) = 0
        ps[i * kBK + c + 8 * jj] = p;
        psum += p;
      }
    }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
    l = l * corr + psum;
    m = m_new;
    __syncthreads();
    const float* pr = ps + i * kBK;
#pragma unroll
    for (int a = 0; a < NACC; ++a) {
      const int e = c + 8 * a;
      float v = acc[a] * corr;
      if (e < vd)
        for (int j = 0; j < nk; ++j) v = fmaf(pr[j], vs[j * vd + e], v);
      acc[a] = v;
    }
    __syncthreads();
  }
  if (q_ok) {
    const float inv = 1.f / l;
#pragma unroll
    for (int a = 0; a < NACC; ++a) {
      const int e = c + 8 * a;
      if (e < vd) out[my_t * ((int64_t)H * vd) + (int64_t)h * vd + e] = rb::from_f<T>(acc[a] * inv);
    }
  }
}

// ------------------------------------------------------------------------------------------------ decode
constexpr int kDT = 128;         // threads per (row, head) CTA
constexpr int kMaxRankRegs = 16; // latent rank <= 32 * 16 = 512

template <typename T>
__global__ void __launch_bounds__(kDT) latent_decode_attention_kernel(
    const T* __restrict__ qc, int64_t ldq, const T* __restrict__ w_ln, const T* __restrict__ w_ukv, T* __restrict__ cache,
    const int* __restrict__ cache_lens, const int* __restrict__ slots, T* __restrict__ out, int H, int qk, int vd, int rank, int R,
    float scale, int window, float eps) {
  extern __shared__ float sm[];
  float* qa = sm;                    // [rank]  query in latent space, times scale
  float* cnew = qa + rank;           // [rank]  this token's latent (own-latent blocks)
  float* accw = cnew + rank;         // [nwarp][rank]
  float* qsm = accw + (kDT / 32) * rank;  // [qk]
  __shared__ float red[32];
  __shared__ float mw[kDT / 32], lw[kDT / 32];
  const int b = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t slot = slots != nullptr ? slots[b] : b;
  const int pos = cache_lens[slot];
  const int n_q = H * qk;
  const bool own = w_ln != nullptr;
  T* crow_new = cache + (slot * R + (pos % R)) * (int64_t)rank;
  if (own) {
    float s = 0.f;
    for (int r = tid; r < rank; r += kDT) { const float v = rb::to_f(qc[b * ldq + n_q + r]); s += v * v; }
    s = rb::block_reduce<false>(s, red);
    const float rstd = 1.f / sqrtf(s / (float)rank + eps);
    for (int r = tid; r < rank; r += kDT) {
      const T v = rb::from_f<T>(rb::to_f(qc[b * ldq + n_q + r]) * rstd * rb::to_f(w_ln[r]));
      cnew[r] = rb::to_f(v);
      if (h == 0) crow_new[r] = v;
    }
  }
  for (int d = tid; d < qk; d += kDT) qsm[d] = rb::to_f(qc[b * ldq + (int64_t)h * qk + d]);
  __syncthreads();
  for (int r = tid; r < rank; r += kDT) {
    float a = 0.f;
    const T* wk = w_ukv + (int64_t)h * qk * rank + r;
    for (int d = 0; d < qk; ++d) a = fmaf(qsm[d], rb::to_f(wk[(int64_t)d * rank]), a);
    qa[r] = a * scale;
  }
  __syncthreads();
  const int reach = (window > 0 && window - 1 < pos) ? window - 1 : pos;
  const int lo = pos - reach;
  float m = -INFINITY, l = 0.f, acc[kMaxRankRegs], crow[kMaxRankRegs];
#pragma unroll
  for (int k = 0; k < kMaxRankRegs; ++k) acc[k] = 0.f;
  for (int j = lo + warp; j <= pos; j += kDT / 32) {
    const bool fresh = own && j == pos;        // the row this launch appends: other CTAs may not have written it yet
    const T* cr = cache + (slot * R + (j % R)) * (int64_t)rank;
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < kMaxRankRegs; ++k) {
      const int r = lane + 32 * k;
      crow[k] = r < rank ? (fresh ? cnew[r] : rb::to_f(cr[r])) : 0.f;
      s = fmaf(crow[k], r < rank ? qa[r] : 0.f, s);
    }
    s = rb::warp_sum(s);
    const float m_new = fmaxf(m, s);
    const float corr = expf(m - m_new), p = expf(s - m_new);
    l = l * corr + p;
    m = m_new;
#pragma unroll
    for (int k = 0; k < kMaxRankRegs; ++k) acc[k] = fmaf(p, crow[k], acc[k] * corr);
  }
  if (lane == 0) { mw[warp] = m; lw[warp] = l; }
#pragma unroll
  for (int k = 0; k < kMaxRankRegs; ++k) {
    const int r = lane + 32 * k;
    if (r < rank) accw[warp * rank + r] = acc[k];
  }
  __syncthreads();
  float M = -INFINITY;
  for (int w_ = 0; w_ < kDT / 32; ++w_) M = fmaxf(M, mw[w_]);
  float L = 0.f;
  for (int w_ = 0; w_ < kDT / 32; ++w_) L += lw[w_] * (mw[w_] == -INFINITY ? 0.f : expf(mw[w_] - M));
  __syncthreads();
  for (int r = tid; r < rank; r += kDT) {     // merged latent-space output, reusing qa
    float o = 0.f;
    for (int w_ = 0; w_ < kDT / 32; ++w_)
      if (mw[w_] != -INFINITY) o += accw[w_ * rank + r] * expf(mw[w_] - M);
    qa[r] = o / L;
  }
  __syncthreads();
  const T* wv = w_ukv + ((int64_t)n_q + (int64_t)h * vd) * rank;
  for (int e = warp; e < vd; e += kDT / 32) {
    float a = 0.f;
    for (int r = lane; r < rank; r += 32) a = fmaf(rb::to_f(wv[(int64_t)e * rank + r]), qa[r], a);
    a = rb::warp_sum(a);
    if (lane == 0) out[(int64_t)b * H * vd + (int64_t)h * vd + e] = rb::from_f<T>(a);
  }
}

template <typename T, int NACC>
int launch_prefill(const void* q, int64_t ldq, const void* kv, int64_t ldkv, const int* pos, void* out, int64_t n_tok, int H, int qk, int vd,
                   float scale, int window, cudaStream_t s) {
  const size_t smem = ((size_t)kBQ * qk + (size_t)kBK * (qk + 1) + (size_t)kBK * vd + (size_t)kBQ * kBK) * sizeof(float);
  if (smem > 200 * 1024) return 1;
  auto kern = latent_window_attention_kernel<T, NACC>;
  if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 2;
  dim3 grid((unsigned)RB_CEIL_DIV(n_tok, (int64_t)kBQ), (unsigned)H);
  kern<<<grid, kPT, smem, s>>>((const T*)q, ldq, (const T*)kv, ldkv, pos, (T*)out, n_tok, H, qk, vd, scale, window);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

template <typename T>
int dispatch_prefill(const void* q, int64_t ldq, const void* kv, int64_t ldkv, const int* pos, void* out, int64_t n_tok, int H, int qk, int vd,
                     float scale, int window, cudaStream_t s) {
  if (vd <= 64) return launch_prefill<T, 8>(q, ldq, kv, ldkv, pos, out, n_tok, H, qk, vd, scale, window, s);
  if (vd <= 128) return launch_prefill<T, 16>(q, ldq, kv, ldkv, pos, out, n_tok, H, qk, vd, scale, window, s);
  if (vd <= 256) return launch_prefill<T, 32>(q, ldq, kv, ldkv, pos, out, n_tok, H, qk, vd, scale, window, s);
  return 1;
}

}  // namespace

#define RB_DISPATCH_T(dt, ...)                                                      \
  switch (dt) {                                                                     \
    case 0: { using T = float; __VA_ARGS__; break; }                                \
    case 1: { using T = __nv_bfloat16; __VA_ARGS__; break; }                        \
    case 2: { using T = __half; __VA_ARGS__; break; }                               \
    default: return 1;                                                              \
  }

extern "C" {

int rb_latent_norm_store(const void* qc, int64_t ldq, int n_q, const void* w, void* c_out, void* cache, const int* tok_slot, const int* pos,
                         const int* remain, int64_t n_tok, int rank, int R, float eps, int dt, cudaStream_t s) {
  if (n_tok == 0) return 0;
  RB_DISPATCH_T(dt, (latent_norm_store_kernel<T><<<(unsigned)RB_CEIL_DIV(n_tok, (int64_t)4), 128, 0, s>>>(
                        (const T*)qc, ldq, n_q, (const T*)w, (T*)c_out, (T*)cache, tok_slot, pos, remain, n_tok, rank, R, eps)));
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int rb_latent_window_attention(const void* q, int64_t ldq, const void* kv, int64_t ldkv, const int* pos, void* out, int64_t n_tok, int H,
                               int qk, int vd, float scale, int window, int dt, cudaStream_t s) {
  if (n_tok == 0) return 0;
  RB_DISPATCH_T(dt, return dispatch_prefill<T>(q, ldq, kv, ldkv, pos, out, n_tok, H, qk, vd, scale, window, s));
  return 1;
}

int rb_latent_decode_attention(const void* qc, int64_t ldq, const void* w_ln, const void* w_ukv, void* cache, const int* cache_lens,
                               const int* slots, void* out, int B, int H, int qk, int vd, int rank, int R, float scale, int window, float eps,
                               int dt, cudaStream_t s) {
  if (B == 0) return 0;
  if (rank > 32 * kMaxRankRegs) return 1;
  const size_t smem = ((size_t)(2 + kDT / 32) * rank + qk) * sizeof(float);
  if (smem > 48 * 1024) return 1;
  dim3 grid((unsigned)B, (unsigned)H);
  RB_DISPATCH_T(dt, (latent_decode_attention_kernel<T><<<grid, kDT, smem, s>>>((const T*)qc, ldq, (const T*)w_ln, (const T*)w_ukv, (T*)cache,
                                                                                cache_lens, slots, (T*)out, H, qk, vd, rank, R, scale, window, eps)));
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
