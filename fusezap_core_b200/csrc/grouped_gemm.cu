// Products over groups with plain 32-bit FMAs: one weight matrix per head (a slice of every row) or per expert (its own
// rows of the step), and the kernel that sorts a step's (row, choice) pairs by expert.
//
// Every output element is one chain of fmaf over k = 0, 1, ..., K-1, started from zero, whichever tile it lands in, so a
// row's result does not depend on the other rows of the step or on where the sort put it.
//
//   heads:    C[m, g, c_off + n] = sum_k A[m, g, a_off + k] * W[g, n, k]          grid (n tiles, row tiles, heads)
//   experts:  tiles (expert, first pair, pairs) written by the sort; row s of a tile reads A[a_idx[s]] (or A[s]) and
//             writes C[c_idx[s]] (or C[s]); with GLU the expert's matrix holds gate rows then up rows and the tile
//             writes act(gate, up) instead of the sums
#include "common.cuh"
#include <math.h>

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

struct GroupedArgs {
  const void* A; long long lda; long long a_group;      // element strides: between rows; between groups (heads mode)
  const void* W; long long w_group;                     // (groups, N or 2N, K) contiguous
  void* C; long long ldc; long long c_group;
  int M, N, K;
  const int* tiles;                                     // experts mode: (group, first, count) per row tile; else null
  const int* a_idx; const int* c_idx;                   // experts mode: row maps (null: identity)
  float alpha, limit, up_shift;                         // GLU: g sigmoid(alpha g) (u + up_shift), g and u clamped by limit
  const int* pad_rows; int pad_n, pad_top;              // experts mode, scatter: rows n with pad_rows[n] < 0 have no
                                                        // pairs; their pad_top output rows are written as zeros
};

template <typename TA, typename TC, bool GLU>
__global__ void __launch_bounds__(256)
grouped_gemm_kernel(const GroupedArgs p) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  __shared__ float Us[GLU ? BK : 1][BN + 4];
  __shared__ int arow_s[BM], crow_s[BM];
  int group, first, count;
  if (p.tiles != nullptr) {
    group = p.tiles[3 * blockIdx.y];
    first = p.tiles[3 * blockIdx.y + 1];
    count = p.tiles[3 * blockIdx.y + 2];
  } else {
    group = blockIdx.z;
    first = blockIdx.y * BM;
    count = min(BM, p.M - first);
  }
  const int tid = threadIdx.x;
  if (p.pad_rows != nullptr && blockIdx.y == 0) {
    for (int n = tid; n < p.pad_n; n += 256) {
      if (p.pad_rows[n] >= 0) continue;
      for (int r = n * p.pad_top; r < (n + 1) * p.pad_top; ++r)
        for (int c = blockIdx.x * BN; c < min(p.N, (int)(blockIdx.x + 1) * BN); ++c)
          ((TC*)p.C)[(long long)r * p.ldc + c] = Cvt<TC>::from_f(0.f);
    }
  }
  if (count <= 0) return;
  if (tid < BM) {
    const int s = first + tid;
    arow_s[tid] = tid < count ? (p.a_idx ? p.a_idx[s] : s) : -1;
    crow_s[tid] = tid < count ? (p.c_idx ? p.c_idx[s] : s) : -1;
  }
  __syncthreads();
  const int tx = tid & 15, ty = tid >> 4;
  const int n0 = blockIdx.x * BN;
  const int lr = tid >> 2, lk = (tid & 3) * 4;
  const int K = p.K, N = p.N;
  const TA* A = (const TA*)p.A + (p.tiles ? 0 : (long long)group * p.a_group);
  const TA* W = (const TA*)p.W + (long long)group * p.w_group;
  const int ar = arow_s[lr];
  const TA* arow = ar >= 0 ? A + (long long)ar * p.lda : nullptr;
  const bool w_ok = n0 + lr < N;
  const TA* wrow = W + (long long)(n0 + lr) * K;
  const TA* urow = wrow + (long long)N * K;      // GLU: the up rows follow the N gate rows

  float acc[TM][TN], acu[GLU ? TM : 1][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      acc[i][j] = 0.f;
      if constexpr (GLU) acu[i][j] = 0.f;
    }
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + lk + i;
      As[lk + i][lr] = (arow != nullptr && k < K) ? Cvt<TA>::to_f(arow[k]) : 0.f;
      Ws[lk + i][lr] = (w_ok && k < K) ? Cvt<TA>::to_f(wrow[k]) : 0.f;
      if constexpr (GLU) Us[lk + i][lr] = (w_ok && k < K) ? Cvt<TA>::to_f(urow[k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN], u[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) {
        b[j] = Ws[kk][tx * TN + j];
        if constexpr (GLU) u[j] = Us[kk][tx * TN + j];
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
          if constexpr (GLU) acu[i][j] = fmaf(a[i], u[j], acu[i][j]);
        }
    }
    __syncthreads();
  }
  TC* C = (TC*)p.C + (p.tiles ? 0 : (long long)group * p.c_group);
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int cr = crow_s[ty * TM + i];
    if (cr < 0) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if constexpr (GLU) {
        const float g = fminf(v, p.limit);
        const float u = fminf(fmaxf(acu[i][j], -p.limit), p.limit);
        v = g * (1.0f / (1.0f + expf(-p.alpha * g))) * (u + p.up_shift);
      }
      C[(long long)cr * p.ldc + n] = Cvt<TC>::from_f(v);
    }
  }
}

// One block sorts the step's N * top (row, choice) pairs by expert. Outputs: a_idx[s] = row and c_idx[s] = row * top +
// choice of the pair at sorted place s; tiles (expert, first place, pairs) for row tiles of tile_rows pairs, the unused ones
// with 0 pairs; rows of padding (seq_row < 0) have no pairs. The order of pairs within an expert is whatever the atomic
// counters give: no result depends on it.
__global__ void __launch_bounds__(1024)
route_by_table_kernel(const int* __restrict__ token_ids, const int* __restrict__ seq_row, const int* __restrict__ table,
                      int N, int V, int top, int E, int* __restrict__ a_idx, int* __restrict__ c_idx,
                      int* __restrict__ tiles, int max_tiles, int tile_rows, int* err) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  extern __shared__ int sm[];
  int* count = sm;            // [E]
  int* start = sm + E;        // [E]
  int* cursor = sm + 2 * E;   // [E]
  for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = cursor[e] = 0;
  __syncthreads();
  const int A = N * top;
  for (int a = threadIdx.x; a < A; a += blockDim.x) {
    const int n = a / top;
    if (seq_row[n] < 0) continue;
    const int tok = token_ids != nullptr ? token_ids[n] : n;      // no ids: row n of the table belongs to row n
    if (tok < 0 || tok >= V) { atomicOr(err, FZ_ERR_TOKEN_RANGE); continue; }
    const int e = table[(size_t)tok * top + (a - n * top)];
    if (e < 0 || e >= E) { atomicOr(err, FZ_ERR_TOKEN_RANGE); continue; }
    atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, t = 0;
    for (int e = 0; e < E; ++e) {
      start[e] = at;
      for (int f = 0; f < count[e] && t < max_tiles; f += tile_rows, ++t) {
        tiles[3 * t] = e;
        tiles[3 * t + 1] = at + f;
        tiles[3 * t + 2] = min(tile_rows, count[e] - f);
      }
      at += count[e];
    }
    for (; t < max_tiles; ++t) tiles[3 * t] = tiles[3 * t + 1] = tiles[3 * t + 2] = 0;
  }
  __syncthreads();
  for (int a = threadIdx.x; a < A; a += blockDim.x) {
    const int n = a / top;
    if (seq_row[n] < 0) continue;
    const int tok = token_ids != nullptr ? token_ids[n] : n;
    if (tok < 0 || tok >= V) continue;
    const int e = table[(size_t)tok * top + (a - n * top)];
    if (e < 0 || e >= E) continue;
    const int s = start[e] + atomicAdd(&cursor[e], 1);
    a_idx[s] = n;
    c_idx[s] = a;
  }
}

template <typename TA, typename TC, bool GLU>
int launch(const GroupedArgs& p, dim3 grid, cudaStream_t stream) {
  fz_launch(grouped_gemm_kernel<TA, TC, GLU>, grid, dim3(256), 0, stream, p);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

int dispatch(const GroupedArgs& p, dim3 grid, int in_dtype, int out_dtype, bool glu, cudaStream_t stream) {
  if (in_dtype == FZ_F32 && out_dtype == FZ_F32) return glu ? launch<float, float, true>(p, grid, stream) : launch<float, float, false>(p, grid, stream);
  if (in_dtype == FZ_BF16 && out_dtype == FZ_BF16) return glu ? launch<__nv_bfloat16, __nv_bfloat16, true>(p, grid, stream) : launch<__nv_bfloat16, __nv_bfloat16, false>(p, grid, stream);
  if (in_dtype == FZ_BF16 && out_dtype == FZ_F32 && !glu) return launch<__nv_bfloat16, float, false>(p, grid, stream);
  return FZ_BAD_DTYPE;
}
}  // namespace

FZ_API int fz_grouped_tile_rows() { return BM; }

// One product per head. A: rows of lda elements, head g at a_off + g * a_head; W: (H, N, K); C likewise.
FZ_API int fz_linear_heads(const void* A, long long lda, long long a_head, const void* W, void* C, long long ldc,
                           long long c_head, int in_dtype, int out_dtype, int M, int H, int N, int K, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || H <= 0) return FZ_OK;
  if (K <= 0) return FZ_BAD_SHAPE;
  if (H > 65535 || (M + BM - 1) / BM > 65535) return FZ_TOO_LARGE;
  GroupedArgs p = {A, lda, a_head, W, (long long)N * K, C, ldc, c_head, M, N, K, nullptr, nullptr, nullptr, 0.f, 0.f, 0.f, nullptr, 0, 0};
  return dispatch(p, dim3((N + BN - 1) / BN, (M + BM - 1) / BM, H), in_dtype, out_dtype, false, stream);
}

FZ_API int fz_route_by_table(const int* token_ids, const int* seq_row, const int* table, int N, int V, int top, int E,
                             int* a_idx, int* c_idx, int* tiles, int max_tiles, int tile_rows, int* err,
                             cudaStream_t stream) {
  if (N <= 0) return FZ_OK;
  if (E <= 0 || E > 4096 || top <= 0 || tile_rows <= 0 || tile_rows > 128) return FZ_BAD_SHAPE;
  fz_launch(route_by_table_kernel, dim3(1), dim3(1024), (size_t)3 * E * sizeof(int), stream, token_ids, seq_row, table, N, V,
            top, E, a_idx, c_idx, tiles, max_tiles, tile_rows, err);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

// Experts mode. glu != 0: W (E, 2N, K), C (pairs, N) in sorted order, A rows through a_idx. glu == 0: W (E, N, K), A
// (pairs, K) in sorted order, C rows through c_idx; pad_rows (may be null): see GroupedArgs.
FZ_API int fz_grouped_linear(const void* A, const void* W, void* C, const int* tiles, int max_tiles, int tile_rows, const int* a_idx,
                             const int* c_idx, int in_dtype, int out_dtype, int N, int K, int glu, float alpha,
                             float limit, float up_shift, const int* pad_rows, int pad_n, int pad_top, cudaStream_t stream) {
  if (max_tiles <= 0 || N <= 0) return FZ_OK;
  if (K <= 0 || tile_rows > BM) return FZ_BAD_SHAPE;      // a tile list built for larger row tiles than this kernel's
  if (max_tiles > 65535) return FZ_TOO_LARGE;
  GroupedArgs p = {A, K, 0, W, (long long)(glu ? 2 : 1) * N * K, C, N, 0, 0, N, K, tiles, a_idx, c_idx, alpha, limit, up_shift, pad_rows, pad_n, pad_top};
  return dispatch(p, dim3((N + BN - 1) / BN, max_tiles, 1), in_dtype, out_dtype, glu != 0, stream);
}

#ifdef FZ_TIMELINE
FZ_TIMELINE_READER(grouped_gemm)
#endif
