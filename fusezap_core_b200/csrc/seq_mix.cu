// Kernels of the recurrent mixers (retention, gated delta rule), of the windowed attention with kept first tokens and a
// sink, and of the routed experts' router and weighted sum. All arithmetic that enters a recurrence, a score, a softmax,
// a norm or a router is 32-bit; T is the activation dtype of what is read or written around them.
//
// Portions: seg[s] = (first row, rows, first position, state slot) per request of the step; a recurrent kernel walks a
// portion's tokens in order from the state in the request's slot and leaves the state there. Nothing depends on which
// other portions share the step.
#include "common.cuh"
#include <math.h>

namespace {
// ------------------------------------------------------------------------------------------ rotation + cache write
// One rotated value of a head: element i of x (dk values), turned by the angle of pair j at position p when i lies in
// the first `rotated` dimensions. pairing 0: (i, i + rotated/2); 1: (2j, 2j + 1).
__device__ __forceinline__ float rotated_value(const float* __restrict__ x, int i, int rotated, int pairing,
                                               const float* __restrict__ cs, const float* __restrict__ sn) {
  if (i >= rotated) return x[i];
  const int half = rotated >> 1;
  int j, a, b;
  if (pairing == 0) { j = i < half ? i : i - half; a = j; b = j + half; }
  else { j = i >> 1; a = 2 * j; b = a + 1; }
  float o1, o2;
  fz_rope_pair(x[a], x[b], cs[j], sn[j], o1, o2);
  return i == a ? o1 : o2;
}

template <typename T>
__global__ void __launch_bounds__(256)
rotate_kv_write_kernel(const float* __restrict__ qkv, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                       int rotated, int pairing, int max_pos, const int* __restrict__ pos, const int* __restrict__ seq_row,
                       const int* __restrict__ table, int mb, T* __restrict__ k_pool, T* __restrict__ v_pool,
                       long long page_stride, long long head_stride, long long tok_stride, int page_size, int n_pages,
                       int write, T* __restrict__ q_out, int Hq, int Hkv, int dk, int dv, int* err) {
  fz_grid_launch_dependents();
  const int n = blockIdx.x;
  const int row = seq_row[n], p = pos[n];      // the step's metadata: written by the host before the step's first kernel
  fz_grid_wait();
  T* qrow = q_out + (size_t)n * Hq * dk;
  if (row < 0 || (rotated > 0 && (p < 0 || p >= max_pos))) {
    if (row >= 0) atomicOr(err, FZ_ERR_POS_RANGE);
    for (int i = threadIdx.x; i < Hq * dk; i += blockDim.x) qrow[i] = Cvt<T>::from_f(0.f);
    return;
  }
  const int width = (Hq + Hkv) * dk + Hkv * dv;
  const float* in = qkv + (size_t)n * width;
  const int half = rotated >> 1;
  const float* cs = cos_t + (size_t)p * half;
  const float* sn = sin_t + (size_t)p * half;
  int page = -1;
  if (write) {
    page = table[(size_t)row * mb + p / page_size];
    if (page < 0 || page >= n_pages) { if (threadIdx.x == 0) atomicOr(err, FZ_ERR_NO_PAGE); page = -1; }
  }
  const long long at = (long long)page * page_stride + (long long)(p % page_size) * tok_stride;
  for (int e = threadIdx.x; e < (Hq + Hkv) * dk; e += blockDim.x) {
    const int head = e / dk, i = e - head * dk;
    const float v = rotated_value(in + (size_t)head * dk, i, rotated, pairing, cs, sn);
    if (head < Hq) qrow[e] = Cvt<T>::from_f(v);
    else if (page >= 0) k_pool[at + (long long)(head - Hq) * head_stride + i] = Cvt<T>::from_f(v);
  }
  if (page >= 0) {
    const float* vin = in + (size_t)(Hq + Hkv) * dk;
    for (int e = threadIdx.x; e < Hkv * dv; e += blockDim.x) {
      const int head = e / dv, i = e - head * dv;
      v_pool[at + (long long)head * head_stride + i] = Cvt<T>::from_f(vin[e]);
    }
  }
}

// ------------------------------------------------------------------------------ attention: window, kept tokens, sink
// One block per (token row, kv head, slice of up to 32 query heads of the kv head's group); warp w serves the query heads
// w, w + W, ... of the slice. Keys are walked in chunks of 32 whose boundaries are multiples of 32 in absolute position,
// first the chunks of the kept first tokens that lie before the window, then the window's, and the running (max, sum,
// accumulator) is updated chunk by chunk; the sink enters last. The order of every sum depends only on the row's own
// position, never on the batch, the cut of the prompt or the pages used.
constexpr int CHUNK = 32;
constexpr int MAX_WARPS = 8;
constexpr int MAX_HPW = 4;
constexpr int MAX_GROUP = MAX_WARPS * MAX_HPW;

template <typename T, int DPL>   // DPL: value dims per lane = ceil(dv / 32)
__global__ void sink_attention_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                                      const int* __restrict__ pos, const int* __restrict__ seq_row,
                                      const int* __restrict__ table, int mb, long long page_stride, long long head_stride,
                                      long long tok_stride, int page_size, int n_pages, T* __restrict__ out, int Hq, int Hkv,
                                      int dk, int dv, float scale, int window, int keep_first,
                                      const float* __restrict__ sink, int* err) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  extern __shared__ float smem[];
  const int n = blockIdx.x, kvh = blockIdx.y;
  const int G_all = Hq / Hkv, g_base = blockIdx.z * MAX_GROUP;
  const int G = min(MAX_GROUP, G_all - g_base);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, W = blockDim.x >> 5;
  const int kstride = dk + 1;
  float* Ks = smem;                       // [CHUNK][dk + 1]
  float* Vs = Ks + CHUNK * kstride;       // [CHUNK][dv]
  float* Qs = Vs + CHUNK * dv;            // [G][dk]
  const int head0 = kvh * G_all + g_base;
  T* orow = out + ((size_t)n * Hq + head0) * dv;
  const int row = seq_row[n];
  if (row < 0) {
    for (int i = threadIdx.x; i < G * dv; i += blockDim.x) orow[i] = Cvt<T>::from_f(0.f);
    return;
  }
  const int p = pos[n];
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int kept = min(keep_first, lo);                      // keys 0 .. kept-1 are seen although they lie before the window
  const T* qrow = q + ((size_t)n * Hq + head0) * dk;
  for (int i = threadIdx.x; i < G * dk; i += blockDim.x) Qs[i] = Cvt<T>::to_f(qrow[i]);

  float m[MAX_HPW], l[MAX_HPW], acc[MAX_HPW][DPL];
#pragma unroll
  for (int a = 0; a < MAX_HPW; ++a) {
    m[a] = -INFINITY;
    l[a] = 0.f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[a][i] = 0.f;
  }
  const int* trow = table + (size_t)row * mb;
  const long long head_off = (long long)kvh * head_stride;
  const int first_end = kept > 0 ? (kept - 1) / CHUNK : -1;      // last chunk of the kept tokens
  const int c2 = max(lo / CHUNK, first_end + 1);                 // first chunk of the window not yet walked
  const int c_last = p / CHUNK;
  for (int it = 0;; ++it) {
    const int c = it <= first_end ? it : c2 + (it - first_end - 1);
    if (c > c_last) break;
    __syncthreads();   // the previous chunk is consumed (and Qs is written, the first time)
    for (int j = warp; j < CHUNK; j += W) {
      const int key = c * CHUNK + j;
      const bool seen = key <= p && (key >= lo || key < kept);
      long long off = -1;
      if (seen) {
        const int page = trow[key / page_size];
        if (page < 0 || page >= n_pages) { if (lane == 0) atomicOr(err, FZ_ERR_NO_PAGE); }
        else off = (long long)page * page_stride + head_off + (long long)(key % page_size) * tok_stride;
      }
      for (int d = lane; d < dk; d += 32) Ks[j * kstride + d] = off >= 0 ? Cvt<T>::to_f(k_pool[off + d]) : 0.f;
      for (int d = lane; d < dv; d += 32) Vs[j * dv + d] = off >= 0 ? Cvt<T>::to_f(v_pool[off + d]) : 0.f;
    }
    __syncthreads();
    const int key = c * CHUNK + lane;
    const bool valid = key <= p && (key >= lo || key < kept);
#pragma unroll
    for (int a = 0; a < MAX_HPW; ++a) {
      const int g = warp + a * W;
      if (g >= G) break;
      const float* qh = Qs + g * dk;
      const float* kr = Ks + lane * kstride;
      float s = 0.f;
      for (int d = 0; d < dk; ++d) s = fmaf(qh[d], kr[d], s);
      s = valid ? s * scale : -INFINITY;
      const float mn = fmaxf(m[a], warp_max(s));       // finite: every chunk walked holds at least one visible key
      const float pj = valid ? expf(s - mn) : 0.f;
      const float corr = expf(m[a] - mn);               // 0 for the first chunk (m = -inf)
      l[a] = l[a] * corr + warp_sum(pj);
      m[a] = mn;
#pragma unroll
      for (int i = 0; i < DPL; ++i) acc[a][i] *= corr;
      for (int j = 0; j < CHUNK; ++j) {
        const float pv = __shfl_sync(0xffffffffu, pj, j);
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
          const int d = lane + 32 * i;
          if (d < dv) acc[a][i] = fmaf(pv, Vs[j * dv + d], acc[a][i]);
        }
      }
    }
  }
#pragma unroll
  for (int a = 0; a < MAX_HPW; ++a) {
    const int g = warp + a * W;
    if (g >= G) break;
    float la = l[a], corr = 1.f;
    if (sink != nullptr) {                  // the sink: one more term of the denominator, no value
      const float sk = sink[head0 + g];
      const float mn = fmaxf(m[a], sk);
      corr = expf(m[a] - mn);
      la = la * corr + expf(sk - mn);
    }
    const float inv = 1.0f / la;
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
      const int d = lane + 32 * i;
      if (d < dv) orow[g * dv + d] = Cvt<T>::from_f(acc[a][i] * corr * inv);
    }
  }
}

// ------------------------------------------------------------------------------------------------ recurrent scans
// The state of a head is a key_dim x value_dim matrix S. A thread owns DPT = 16 consecutive rows of one column; the R
// lanes that share a column (R a power of two, R * 16 >= key_dim, neighbours in a warp) add their partial dot products
// with shuffles. State layout in memory: (slots, heads, value_dim, R * 16), so a thread's 16 values are contiguous and a
// warp reads one contiguous run; rows beyond key_dim stay zero. A block of 256 threads covers 256 / R columns of one
// head of one portion and walks the portion's tokens in chunks of TCH, staged in shared memory by all threads.
constexpr int DPT = 16;
constexpr int TCH = 8;
constexpr int SCAN_THREADS = 256;

__device__ __forceinline__ float lanes_sum(float v, int R) {
  for (int o = R >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ void load_state(const float* __restrict__ p, float* S) {
#pragma unroll
  for (int i = 0; i < DPT; i += 4) {
    const float4 v = *(const float4*)(p + i);
    S[i] = v.x; S[i + 1] = v.y; S[i + 2] = v.z; S[i + 3] = v.w;
  }
}
__device__ __forceinline__ void store_state(float* __restrict__ p, const float* S) {
#pragma unroll
  for (int i = 0; i < DPT; i += 4) *(float4*)(p + i) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
}

// S = decay * S + k' v^T; o = S^T q'. proj rows: [q heads | k heads | v heads | ...], ld floats apart.
__global__ void __launch_bounds__(SCAN_THREADS)
retention_scan_kernel(const float* __restrict__ proj, int ld, int H, int dk, int dv, int R, const float* __restrict__ decay,
                      float key_scale, const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rotated,
                      int pairing, int max_pos, float* __restrict__ state, const int* __restrict__ seg,
                      float* __restrict__ out, int* err) {
  fz_grid_launch_dependents();
  const int s = blockIdx.x, h = blockIdx.y;
  const int row0 = seg[4 * s], cnt = seg[4 * s + 1], pos0 = seg[4 * s + 2], slot = seg[4 * s + 3];
  fz_grid_wait();
  if (cnt <= 0 || slot < 0) return;
  if (rotated > 0 && (pos0 < 0 || pos0 + cnt > max_pos)) { if (threadIdx.x == 0) atomicOr(err, FZ_ERR_POS_RANGE); return; }
  extern __shared__ float smem[];
  const int dkp = R * DPT, COLS = SCAN_THREADS / R;
  float* qs = smem;                    // [TCH][dkp]
  float* ks = qs + TCH * dkp;          // [TCH][dkp]
  float* vs = ks + TCH * dkp;          // [TCH][COLS]
  const int cl = threadIdx.x / R, r = threadIdx.x - cl * R;
  const int col = blockIdx.z * COLS + cl;
  const bool live = col < dv;
  float* sp = state + (((size_t)slot * H + h) * dv + (live ? col : 0)) * dkp + r * DPT;
  float S[DPT];
  if (live) load_state(sp, S);
  else {
#pragma unroll
    for (int i = 0; i < DPT; ++i) S[i] = 0.f;
  }
  const float dec = decay[h];
  const int half = rotated >> 1;
  for (int t0 = 0; t0 < cnt; t0 += TCH) {
    const int tc = min(TCH, cnt - t0);
    __syncthreads();
    for (int e = threadIdx.x; e < tc * dkp; e += SCAN_THREADS) {
      const int tt = e / dkp, i = e - tt * dkp;
      float qv = 0.f, kv = 0.f;
      if (i < dk) {
        const float* in = proj + (size_t)(row0 + t0 + tt) * ld;
        const size_t at = (size_t)(pos0 + t0 + tt) * half;
        qv = rotated_value(in + (size_t)h * dk, i, rotated, pairing, cos_t + at, sin_t + at);
        kv = __fmul_rn(rotated_value(in + (size_t)(H + h) * dk, i, rotated, pairing, cos_t + at, sin_t + at), key_scale);
      }
      qs[e] = qv;
      ks[e] = kv;
    }
    for (int e = threadIdx.x; e < tc * COLS; e += SCAN_THREADS) {
      const int tt = e / COLS, c = e - tt * COLS;
      const int cc = blockIdx.z * COLS + c;
      vs[e] = cc < dv ? proj[(size_t)(row0 + t0 + tt) * ld + (size_t)2 * H * dk + (size_t)h * dv + cc] : 0.f;
    }
    __syncthreads();
    for (int tt = 0; tt < tc; ++tt) {
      const float v = vs[tt * COLS + cl];
      const float* kk = ks + tt * dkp + r * DPT;
      const float* qq = qs + tt * dkp + r * DPT;
      float o = 0.f;
#pragma unroll
      for (int i = 0; i < DPT; ++i) {
        S[i] = __fmaf_rn(dec, S[i], __fmul_rn(kk[i], v));
        o = __fmaf_rn(S[i], qq[i], o);
      }
      o = lanes_sum(o, R);
      if (live && r == 0) out[(size_t)(row0 + t0 + tt) * H * dv + (size_t)h * dv + col] = o;
    }
  }
  if (live) store_state(sp, S);
}

// S = g * S (rows); u = beta (v - S^T k^); S += k^ u^T; o = S^T q^. qkv rows: [q (Hk dk) | k (Hk dk) | v (H dv)] of T.
template <typename T>
__global__ void __launch_bounds__(SCAN_THREADS)
gated_delta_scan_kernel(const T* __restrict__ qkv, int H, int Hk, int dk, int dv, int R, const float* __restrict__ high,
                        int ldh, const float* __restrict__ beta, const float* __restrict__ a_log,
                        const float* __restrict__ dt_bias, float unit_eps, float q_scale, float* __restrict__ state,
                        const int* __restrict__ seg, float* __restrict__ out) {
  fz_grid_launch_dependents();
  const int s = blockIdx.x, h = blockIdx.y;
  const int row0 = seg[4 * s], cnt = seg[4 * s + 1], slot = seg[4 * s + 3];
  fz_grid_wait();
  if (cnt <= 0 || slot < 0) return;
  extern __shared__ float smem[];
  const int dkp = R * DPT, COLS = SCAN_THREADS / R;
  float* qs = smem;                    // [TCH][dkp]
  float* ks = qs + TCH * dkp;
  float* gs = ks + TCH * dkp;
  float* vs = gs + TCH * dkp;          // [TCH][COLS]
  float* bs = vs + TCH * COLS;         // [TCH]
  const int cl = threadIdx.x / R, r = threadIdx.x - cl * R;
  const int col = blockIdx.z * COLS + cl;
  const bool live = col < dv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kh = h / (H / Hk);
  const int C = 2 * Hk * dk + H * dv;
  float* sp = state + (((size_t)slot * H + h) * dv + (live ? col : 0)) * dkp + r * DPT;
  float S[DPT];
  if (live) load_state(sp, S);
  else {
#pragma unroll
    for (int i = 0; i < DPT; ++i) S[i] = 0.f;
  }
  const float rate = expf(a_log[h]);
  for (int t0 = 0; t0 < cnt; t0 += TCH) {
    const int tc = min(TCH, cnt - t0);
    __syncthreads();
    for (int tt = warp; tt < tc; tt += SCAN_THREADS / 32) {      // a warp stages a token: unit vectors, decays, beta
      const size_t n = (size_t)(row0 + t0 + tt);
      const T* qin = qkv + n * C + (size_t)kh * dk;
      const T* kin = qin + (size_t)Hk * dk;
      float sq = 0.f, sk = 0.f;
      for (int i = lane; i < dk; i += 32) {
        const float a = Cvt<T>::to_f(qin[i]), b = Cvt<T>::to_f(kin[i]);
        sq = fmaf(a, a, sq);
        sk = fmaf(b, b, sk);
      }
      const float nq = sqrtf(warp_sum(sq) + unit_eps), nk = sqrtf(warp_sum(sk) + unit_eps);
      for (int i = lane; i < dkp; i += 32) {
        float qv = 0.f, kv = 0.f, gv = 0.f;
        if (i < dk) {
          qv = __fmul_rn(__fdiv_rn(Cvt<T>::to_f(qin[i]), nq), q_scale);
          kv = __fdiv_rn(Cvt<T>::to_f(kin[i]), nk);
          const float a = high[n * ldh + (size_t)h * dk + i] + dt_bias[(size_t)h * dk + i];
          const float soft = a > 20.f ? a : log1pf(expf(a));
          gv = expf(-rate * soft);
        }
        qs[tt * dkp + i] = qv;
        ks[tt * dkp + i] = kv;
        gs[tt * dkp + i] = gv;
      }
      if (lane == 0) bs[tt] = 1.0f / (1.0f + expf(-beta[n * H + h]));
    }
    for (int e = threadIdx.x; e < tc * COLS; e += SCAN_THREADS) {
      const int tt = e / COLS, c = e - tt * COLS;
      const int cc = blockIdx.z * COLS + c;
      vs[e] = cc < dv ? Cvt<T>::to_f(qkv[(size_t)(row0 + t0 + tt) * C + (size_t)2 * Hk * dk + (size_t)h * dv + cc]) : 0.f;
    }
    __syncthreads();
    for (int tt = 0; tt < tc; ++tt) {
      const float v = vs[tt * COLS + cl], b = bs[tt];
      const float* kk = ks + tt * dkp + r * DPT;
      const float* qq = qs + tt * dkp + r * DPT;
      const float* gg = gs + tt * dkp + r * DPT;
      float ksum = 0.f;
#pragma unroll
      for (int i = 0; i < DPT; ++i) {
        S[i] = __fmul_rn(gg[i], S[i]);
        ksum = __fmaf_rn(S[i], kk[i], ksum);
      }
      ksum = lanes_sum(ksum, R);
      const float u = __fmul_rn(b, v - ksum);
      float o = 0.f;
#pragma unroll
      for (int i = 0; i < DPT; ++i) {
        S[i] = __fmaf_rn(kk[i], u, S[i]);
        o = __fmaf_rn(S[i], qq[i], o);
      }
      o = lanes_sum(o, R);
      if (live && r == 0) out[(size_t)(row0 + t0 + tt) * H * dv + (size_t)h * dv + col] = o;
    }
  }
  if (live) store_state(sp, S);
}

// out[n, h, c] = o / sqrt(mean_c o^2 + eps) * w[c] * act(gate[n, goff + h dv + c]); a warp per (row, head).
template <typename TO>
__global__ void __launch_bounds__(256)
head_norm_gate_kernel(const float* __restrict__ o, int H, int dv, const float* __restrict__ w, float eps,
                      const float* __restrict__ gate, int ldg, int goff, int act, const int* __restrict__ seq_row,
                      TO* __restrict__ out) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  const int n = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, W = blockDim.x >> 5;
  const bool pad = seq_row[n] < 0;
  for (int h = warp; h < H; h += W) {
    const float* x = o + ((size_t)n * H + h) * dv;
    TO* y = out + ((size_t)n * H + h) * dv;
    if (pad) {
      for (int c = lane; c < dv; c += 32) y[c] = Cvt<TO>::from_f(0.f);
      continue;
    }
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) ss = fmaf(x[c], x[c], ss);
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)dv + eps);
    for (int c = lane; c < dv; c += 32) {
      float v = x[c] * inv;
      if (w != nullptr) v *= w[c];
      if (gate != nullptr) {
        const float z = gate[(size_t)n * ldg + goff + (size_t)h * dv + c];
        const float sg = 1.0f / (1.0f + expf(-z));
        v *= act == 2 ? z * sg : sg;
      }
      y[c] = Cvt<TO>::from_f(v);
    }
  }
}

// ------------------------------------------------------------------------------------------------ router
// A warp per row: softmax over the E router logits, then lane 0 picks the groups and the experts. Scores of chosen
// experts are overwritten with -1 in shared memory (scores are never negative), so each is picked once.
constexpr int ROUTER_WARPS = 4;
__global__ void __launch_bounds__(32 * ROUTER_WARPS)
router_topk_kernel(const float* __restrict__ logits, int ld, int N, int E, int top, int groups, int keep, int renorm,
                   const int* __restrict__ seq_row, int* __restrict__ choice, float* __restrict__ weight) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * ROUTER_WARPS + warp;
  if (n >= N) return;
  float* s = smem + (size_t)warp * (E + groups);
  float* gmax = s + E;
  if (seq_row[n] < 0) {
    for (int k = lane; k < top; k += 32) { choice[(size_t)n * top + k] = 0; weight[(size_t)n * top + k] = 0.f; }
    return;
  }
  const float* z = logits + (size_t)n * ld;
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) { const float v = expf(z[e] - mx); s[e] = v; sum += v; }
  sum = warp_sum(sum);
  __syncwarp();
  for (int e = lane; e < E; e += 32) s[e] = __fdiv_rn(s[e], sum);
  __syncwarp();
  const int per = E / groups;
  for (int g = lane; g < groups; g += 32) {
    float v = -1.f;
    for (int e = g * per; e < (g + 1) * per; ++e) v = fmaxf(v, s[e]);
    gmax[g] = v;
  }
  __syncwarp();
  if (lane == 0) {
    // the groups that are not kept lose their experts: groups - keep times, strike the worst group (the higher index
    // among equals, so that the lower index stays)
    for (int d = 0; d < groups - keep; ++d) {
      int worst = -1;
      float wv = 0.f;
      for (int g = 0; g < groups; ++g) {
        if (gmax[g] < -1.5f) continue;                 // already struck
        if (worst < 0 || !(gmax[g] > wv)) { worst = g; wv = gmax[g]; }
      }
      gmax[worst] = -2.f;
      for (int e = worst * per; e < (worst + 1) * per; ++e) s[e] = -1.f;
    }
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
      int best = -1;
      float bv = -1.f;
      for (int e = 0; e < E; ++e)
        if (s[e] > bv) { best = e; bv = s[e]; }
      if (best < 0) {                                  // scores that are not numbers: any expert not yet taken
        for (int e = 0; e < E && best < 0; ++e)
          if (!(s[e] == -1.f)) best = e;
        if (best < 0) best = 0;
        bv = 0.f;
      }
      choice[(size_t)n * top + k] = best;
      weight[(size_t)n * top + k] = bv;
      total += bv;
      s[best] = -1.f;
    }
    if (renorm)
      for (int k = 0; k < top; ++k) weight[(size_t)n * top + k] = __fdiv_rn(weight[(size_t)n * top + k], total);
  }
}

// out[n] = sum_k w[n, k] terms[n top + k] (+ sigmoid(gl[n, col]) shared[n]); rows of padding give zeros.
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ terms, const float* __restrict__ w, int top, const float* __restrict__ shared,
                   const float* __restrict__ gl, int ldg, int col, const int* __restrict__ seq_row, float* __restrict__ out,
                   int N, int D) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  const int n = blockIdx.x;
  const bool pad = seq_row[n] < 0;
  float sg = 0.f;
  if (!pad && shared != nullptr) sg = 1.0f / (1.0f + expf(-gl[(size_t)n * ldg + col]));
  for (int d = blockIdx.y * blockDim.x + threadIdx.x; d < D; d += gridDim.y * blockDim.x) {
    float acc = 0.f;
    if (!pad) {
      for (int k = 0; k < top; ++k) acc = __fmaf_rn(w[(size_t)n * top + k], terms[((size_t)n * top + k) * D + d], acc);
      if (shared != nullptr) acc = __fmaf_rn(sg, shared[(size_t)n * D + d], acc);
    }
    out[(size_t)n * D + d] = acc;
  }
}

struct Terms {
  const float* t[4];
  float w[4];
  int n;
};
__global__ void __launch_bounds__(256) weighted_sum_kernel(const Terms p, float* __restrict__ out, size_t total) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    float acc = __fmul_rn(p.w[0], p.t[0][i]);
    for (int k = 1; k < p.n; ++k) acc = __fadd_rn(acc, __fmul_rn(p.w[k], p.t[k][i]));
    out[i] = acc;
  }
}

int lanes_per_column(int dk) {
  int R = 1;
  while (R * DPT < dk) R <<= 1;
  return R;
}

template <typename T, int DPL>
int launch_sink(const void* q, const void* k_pool, const void* v_pool, const int* pos, const int* seq_row, const int* table,
                int mb, long long page_stride, long long head_stride, long long tok_stride, int page_size, int n_pages,
                void* out, int N, int Hq, int Hkv, int dk, int dv, float scale, int window, int keep_first,
                const float* sink, int* err, cudaStream_t stream) {
  const int G_all = Hq / Hkv, G = G_all < MAX_GROUP ? G_all : MAX_GROUP;
  const int W = G < MAX_WARPS ? G : MAX_WARPS;
  const size_t smem = sizeof(float) * ((size_t)CHUNK * (dk + 1) + (size_t)CHUNK * dv + (size_t)G * dk);
  auto kern = sink_attention_kernel<T, DPL>;
  static size_t allowed = 48 * 1024;
  if (smem > allowed) {
    if (smem > 227 * 1024) return FZ_TOO_LARGE;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    allowed = smem;
  }
  dim3 grid(N, Hkv, (G_all + MAX_GROUP - 1) / MAX_GROUP);
  fz_launch(kern, grid, dim3(32 * W), smem, stream, (const T*)q, (const T*)k_pool, (const T*)v_pool, pos, seq_row, table, mb,
            page_stride, head_stride, tok_stride, page_size, n_pages, (T*)out, Hq, Hkv, dk, dv, scale, window, keep_first,
            sink, err);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

template <typename T>
int dispatch_sink(const void* q, const void* k_pool, const void* v_pool, const int* pos, const int* seq_row,
                  const int* table, int mb, long long page_stride, long long head_stride, long long tok_stride,
                  int page_size, int n_pages, void* out, int N, int Hq, int Hkv, int dk, int dv, float scale, int window,
                  int keep_first, const float* sink, int* err, cudaStream_t stream) {
#define FZ_GO(D) return launch_sink<T, D>(q, k_pool, v_pool, pos, seq_row, table, mb, page_stride, head_stride, tok_stride, page_size, n_pages, out, N, Hq, Hkv, dk, dv, scale, window, keep_first, sink, err, stream)
  const int dpl = (dv + 31) / 32;
  if (dpl <= 1) FZ_GO(1);
  if (dpl <= 2) FZ_GO(2);
  if (dpl <= 4) FZ_GO(4);
  if (dpl <= 8) FZ_GO(8);
  if (dpl <= 16) FZ_GO(16);
#undef FZ_GO
  return FZ_BAD_SHAPE;
}
}  // namespace

FZ_API int fz_rotate_kv_write(const float* qkv, const float* cos_t, const float* sin_t, int rotated, int pairing, int max_pos,
                              const int* pos, const int* seq_row, const int* table, int mb, void* k_pool, void* v_pool,
                              long long page_stride, long long head_stride, long long tok_stride, int page_size,
                              int n_pages, int write, void* q_out, int dtype, int N, int Hq, int Hkv, int dk, int dv, int* err,
                              cudaStream_t stream) {
  if (N <= 0) return FZ_OK;
  if (rotated < 0 || rotated > dk || (rotated & 1) || page_size <= 0 || Hq <= 0 || Hkv <= 0 || dk <= 0 || dv <= 0) return FZ_BAD_SHAPE;
  if (dtype == FZ_F32)
    fz_launch(rotate_kv_write_kernel<float>, dim3(N), dim3(256), 0, stream, qkv, cos_t, sin_t, rotated, pairing, max_pos, pos,
              seq_row, table, mb, (float*)k_pool, (float*)v_pool, page_stride, head_stride, tok_stride, page_size, n_pages,
              write, (float*)q_out, Hq, Hkv, dk, dv, err);
  else if (dtype == FZ_BF16)
    fz_launch(rotate_kv_write_kernel<__nv_bfloat16>, dim3(N), dim3(256), 0, stream, qkv, cos_t, sin_t, rotated, pairing, max_pos,
              pos, seq_row, table, mb, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, page_stride, head_stride, tok_stride,
              page_size, n_pages, write, (__nv_bfloat16*)q_out, Hq, Hkv, dk, dv, err);
  else return FZ_BAD_DTYPE;
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

// Sizes taken: Hq any multiple of Hkv, 0 < dk, dv <= 512.
FZ_API int fz_sink_attention_check(int Hq, int Hkv, int dk, int dv) {
  if (Hq <= 0 || Hkv <= 0 || dk <= 0 || dv <= 0 || Hq % Hkv || dk > 512 || dv > 512 || Hkv > 65535) return FZ_BAD_SHAPE;
  if ((Hq / Hkv + MAX_GROUP - 1) / MAX_GROUP > 65535) return FZ_BAD_SHAPE;
  return FZ_OK;
}

FZ_API int fz_sink_attention(const void* q, const void* k_pool, const void* v_pool, const int* pos, const int* seq_row,
                             const int* table, int mb, long long page_stride, long long head_stride, long long tok_stride,
                             int page_size, int n_pages, void* out, int dtype, int N, int Hq, int Hkv, int dk, int dv,
                             float scale, int window, int keep_first, const float* sink, int* err, cudaStream_t stream) {
  if (N <= 0) return FZ_OK;
  if (fz_sink_attention_check(Hq, Hkv, dk, dv) != FZ_OK || page_size <= 0 || window < 0 || keep_first < 0) return FZ_BAD_SHAPE;
  if (dtype == FZ_F32)
    return dispatch_sink<float>(q, k_pool, v_pool, pos, seq_row, table, mb, page_stride, head_stride, tok_stride, page_size,
                                n_pages, out, N, Hq, Hkv, dk, dv, scale, window, keep_first, sink, err, stream);
  if (dtype == FZ_BF16)
    return dispatch_sink<__nv_bfloat16>(q, k_pool, v_pool, pos, seq_row, table, mb, page_stride, head_stride, tok_stride,
                                        page_size, n_pages, out, N, Hq, Hkv, dk, dv, scale, window, keep_first, sink, err, stream);
  return FZ_BAD_DTYPE;
}

// The padded key size of the recurrent state, (slots, heads, value_dim, this): 16 times a power of two, at most 512.
FZ_API int fz_recurrent_key_pad(int dk) {
  if (dk <= 0 || dk > 512) return -1;
  return lanes_per_column(dk) * DPT;
}

FZ_API int fz_retention_scan(const float* proj, int ld, int H, int dk, int dv, const float* decay, float key_scale,
                             const float* cos_t, const float* sin_t, int rotated, int pairing, int max_pos, float* state,
                             const int* seg, int n_seg, float* out, int* err, cudaStream_t stream) {
  if (n_seg <= 0) return FZ_OK;
  if (H <= 0 || H > 65535 || dv <= 0 || fz_recurrent_key_pad(dk) < 0 || rotated < 0 || rotated > dk || (rotated & 1)) return FZ_BAD_SHAPE;
  const int R = lanes_per_column(dk), cols = SCAN_THREADS / R;
  const size_t smem = sizeof(float) * ((size_t)2 * TCH * R * DPT + (size_t)TCH * cols);
  fz_launch(retention_scan_kernel, dim3(n_seg, H, (dv + cols - 1) / cols), dim3(SCAN_THREADS), smem, stream, proj, ld, H, dk, dv,
            R, decay, key_scale, cos_t, sin_t, rotated, pairing, max_pos, state, seg, out, err);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

FZ_API int fz_gated_delta_scan(const void* qkv, int dtype, int H, int Hk, int dk, int dv, const float* high, int ldh,
                               const float* beta, const float* a_log, const float* dt_bias, float unit_eps, float q_scale,
                               float* state, const int* seg, int n_seg, float* out, cudaStream_t stream) {
  if (n_seg <= 0) return FZ_OK;
  if (H <= 0 || H > 65535 || Hk <= 0 || H % Hk || dv <= 0 || fz_recurrent_key_pad(dk) < 0) return FZ_BAD_SHAPE;
  const int R = lanes_per_column(dk), cols = SCAN_THREADS / R;
  const size_t smem = sizeof(float) * ((size_t)3 * TCH * R * DPT + (size_t)TCH * cols + TCH);
  if (smem > 48 * 1024) return FZ_TOO_LARGE;
  const dim3 grid(n_seg, H, (dv + cols - 1) / cols);
  if (dtype == FZ_F32)
    fz_launch(gated_delta_scan_kernel<float>, grid, dim3(SCAN_THREADS), smem, stream, (const float*)qkv, H, Hk, dk, dv, R, high,
              ldh, beta, a_log, dt_bias, unit_eps, q_scale, state, seg, out);
  else if (dtype == FZ_BF16)
    fz_launch(gated_delta_scan_kernel<__nv_bfloat16>, grid, dim3(SCAN_THREADS), smem, stream, (const __nv_bfloat16*)qkv, H, Hk,
              dk, dv, R, high, ldh, beta, a_log, dt_bias, unit_eps, q_scale, state, seg, out);
  else return FZ_BAD_DTYPE;
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

// act: 0 none, 1 sigmoid, 2 silu.
FZ_API int fz_head_norm_gate(const float* o, int N, int H, int dv, const float* w, float eps, const float* gate, int ldg,
                             int goff, int act, const int* seq_row, void* out, int out_dtype, cudaStream_t stream) {
  if (N <= 0) return FZ_OK;
  if (H <= 0 || dv <= 0) return FZ_BAD_SHAPE;
  const int W = H < 8 ? H : 8;
  if (out_dtype == FZ_F32)
    fz_launch(head_norm_gate_kernel<float>, dim3(N), dim3(32 * W), 0, stream, o, H, dv, w, eps, gate, ldg, goff, act, seq_row, (float*)out);
  else if (out_dtype == FZ_BF16)
    fz_launch(head_norm_gate_kernel<__nv_bfloat16>, dim3(N), dim3(32 * W), 0, stream, o, H, dv, w, eps, gate, ldg, goff, act, seq_row, (__nv_bfloat16*)out);
  else return FZ_BAD_DTYPE;
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

FZ_API int fz_router_topk(const float* logits, int ld, int N, int E, int top, int groups, int keep, int renorm,
                          const int* seq_row, int* choice, float* weight, cudaStream_t stream) {
  if (N <= 0) return FZ_OK;
  if (E <= 0 || E > 2048 || top <= 0 || top > E || groups <= 0 || E % groups || keep <= 0 || keep > groups ||
      top > keep * (E / groups)) return FZ_BAD_SHAPE;
  const size_t smem = sizeof(float) * ROUTER_WARPS * (size_t)(E + groups);
  fz_launch(router_topk_kernel, dim3((N + ROUTER_WARPS - 1) / ROUTER_WARPS), dim3(32 * ROUTER_WARPS), smem, stream, logits, ld,
            N, E, top, groups, keep, renorm, seq_row, choice, weight);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

FZ_API int fz_moe_combine(const float* terms, const float* w, int top, const float* shared, const float* gl, int ldg, int col,
                          const int* seq_row, float* out, int N, int D, cudaStream_t stream) {
  if (N <= 0 || D <= 0) return FZ_OK;
  const int by = (D + 1023) / 1024 > 0 ? (D + 1023) / 1024 : 1;
  fz_launch(moe_combine_kernel, dim3(N, by), dim3(256), 0, stream, terms, w, top, shared, gl, ldg, col, seq_row, out, N, D);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

FZ_API int fz_weighted_sum(const float* t0, const float* t1, const float* t2, const float* t3, float w0, float w1, float w2,
                           float w3, int n_terms, float* out, long long total, cudaStream_t stream) {
  if (total <= 0) return FZ_OK;
  if (n_terms < 1 || n_terms > 4) return FZ_BAD_SHAPE;
  Terms p = {{t0, t1, t2, t3}, {w0, w1, w2, w3}, n_terms};
  const long long blocks = (total + 255) / 256;
  fz_launch(weighted_sum_kernel, dim3((unsigned)(blocks < 65535 ? blocks : 65535)), dim3(256), 0, stream, p, out, (size_t)total);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

#ifdef FZ_TIMELINE
FZ_TIMELINE_READER(seq_mix)
#endif
