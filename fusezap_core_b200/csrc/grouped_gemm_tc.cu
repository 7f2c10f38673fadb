// Products over groups on tensor cores (bf16, mma.sync m16n8k16, float32 accumulation): one weight matrix per head (a
// slice of every row) or per expert (its own rows of the step, gathered and scattered through index lists), with the
// gated activation of the experts computed from the unrounded sums. Same meanings and the same tile lists as the plain
// kernels of grouped_gemm.cu; a row's result does not depend on the tile it lands in (every output is the sum over k in
// the fixed order of the 16-wide MMA steps).
//
// A block computes ROWS x 64 outputs, k in slices of 32 (64 for the 16-row tiles) through a three-stage cp.async ring. ROWS = 64 (four warps) or
// 128 (eight): warp w owns 32 rows (32 (w / 2) ..) and 32 columns (32 (w % 2) ..), so a 16-wide k step takes two
// ldmatrix of A and two of W for eight MMAs (a warp that owned 16 rows and all 64 columns took one and four: the
// shared-memory pipe, not the tensor pipe, was the busier one). Many rows per group: prompts. ROWS = 16: each of four
// warps owns the 16 rows and 16 of the columns (few rows per group: decoded tokens, where the weights are read once
// whatever the rows).
// Shared-memory rows are 16 bytes longer than a slice (80 or 144 bytes: the eight rows of an ldmatrix fall into
// different banks).
//
// Needs K % 8 == 0, N even, and 16-byte aligned rows of A and W; everything else goes to the plain kernel.
#include "attn_mma.cuh"
#include <math.h>

namespace {
using namespace fzattn;

constexpr int BN = 64, STAGES = 3;
// k per slice: 32 for the many-row tiles, 64 for the 16-row tiles (measured at width 2,048: the few-row products of a
// decode step 42 -> 34 us and 23 -> 18 us with 64, the many-row products of a prompt 319 -> 350 us)
template <int ROWS> struct Slice {
  static constexpr int BK = ROWS == 16 ? 64 : 32;
  static constexpr int SROW = BK + 8;       // shared-memory row: 16 bytes more than the slice, so ldmatrix rows spread over the banks
  static constexpr int CH = BK / 8;         // 16-byte chunks per row of a slice
};

struct GroupedArgs {
  const __nv_bfloat16* A; long long lda; long long a_group;
  const __nv_bfloat16* W; long long w_group;
  void* C; long long ldc; long long c_group;
  int M, N, K;
  const int* tiles; const int* a_idx; const int* c_idx;
  float alpha, limit, up_shift;
  const int* pad_rows; int pad_n, pad_top;
};

template <typename TC> __device__ __forceinline__ void store2(TC* p, float a, float b);
template <> __device__ __forceinline__ void store2<float>(float* p, float a, float b) { *(float2*)p = make_float2(a, b); }
template <> __device__ __forceinline__ void store2<__nv_bfloat16>(__nv_bfloat16* p, float a, float b) { *(uint32_t*)p = pack_bf16(a, b); }

template <int ROWS, typename TC, bool GLU>
__global__ void __launch_bounds__(ROWS == 128 ? 256 : 128)
grouped_gemm_tc_kernel(const GroupedArgs p) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  constexpr int THREADS = ROWS == 128 ? 256 : 128;
  constexpr int BK = Slice<ROWS>::BK, SROW = Slice<ROWS>::SROW, CH = Slice<ROWS>::CH;
  constexpr int WCOLS = ROWS >= 64 ? 32 : 16;         // columns a warp owns
  constexpr int NB = WCOLS / 8;                       // 8-column blocks per warp
  constexpr int MB = ROWS >= 64 ? 2 : 1;              // 16-row blocks per warp
  constexpr int A_BYTES = ROWS * SROW * 2, W_BYTES = BN * SROW * 2, STAGE = A_BYTES + (GLU ? 2 : 1) * W_BYTES;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ int arow_s[ROWS], crow_s[ROWS];
  const uint32_t s0 = smem_u32(smem);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int group, first, count;
  if (p.tiles != nullptr) {
    group = p.tiles[3 * blockIdx.y];
    first = p.tiles[3 * blockIdx.y + 1];
    count = p.tiles[3 * blockIdx.y + 2];
  } else {
    group = blockIdx.z;
    first = blockIdx.y * ROWS;
    count = min(ROWS, p.M - first);
  }
  const int n0 = blockIdx.x * BN;
  if (p.pad_rows != nullptr && blockIdx.y == 0) {
    for (int n = tid; n < p.pad_n; n += THREADS) {
      if (p.pad_rows[n] >= 0) continue;
      for (int r = n * p.pad_top; r < (n + 1) * p.pad_top; ++r)
        for (int c = n0; c < min(p.N, n0 + BN); ++c) ((TC*)p.C)[(long long)r * p.ldc + c] = (TC)0.f;
    }
  }
  if (count <= 0) return;
  if (tid < ROWS) {
    const int s = first + tid;
    arow_s[tid] = tid < count ? (p.a_idx ? p.a_idx[s] : s) : -1;
    crow_s[tid] = tid < count ? (p.c_idx ? p.c_idx[s] : s) : -1;
  }
  __syncthreads();
  const int K = p.K, N = p.N;
  const __nv_bfloat16* A = p.A + (p.tiles ? 0 : (long long)group * p.a_group);
  const __nv_bfloat16* W = p.W + (long long)group * p.w_group;
  const int ksl = (K + BK - 1) / BK;

  auto issue = [&](int t) {
    const uint32_t st = s0 + (t % STAGES) * STAGE;
    const int k0 = t * BK;
    // A: ROWS rows x CH chunks of 8; W (and the up rows): 64 rows x CH chunks
    for (int e = tid; e < ROWS * CH; e += THREADS) {
      const int r = e / CH, c = e % CH;
      const int ar = arow_s[r];
      const bool ok = ar >= 0 && k0 + c * 8 < K;
      cp_async16(st + r * SROW * 2 + c * 16, ok ? A + (long long)ar * p.lda + k0 + c * 8 : A, ok);
    }
    for (int e = tid; e < BN * CH; e += THREADS) {
      const int r = e / CH, c = e % CH;
      const bool ok = n0 + r < N && k0 + c * 8 < K;
      const __nv_bfloat16* src = W + (long long)(n0 + r) * K + k0 + c * 8;
      cp_async16(st + A_BYTES + r * SROW * 2 + c * 16, ok ? src : W, ok);
      if constexpr (GLU) cp_async16(st + A_BYTES + W_BYTES + r * SROW * 2 + c * 16, ok ? src + (long long)N * K : W, ok);
    }
    cp_async_commit();
  };
#pragma unroll
  for (int t = 0; t < STAGES - 1; ++t) {
    if (t < ksl) issue(t); else cp_async_commit();
  }
  float acc[MB][NB][4], acu[GLU ? MB : 1][GLU ? NB : 1][4];
#pragma unroll
  for (int m = 0; m < MB; ++m)
#pragma unroll
    for (int j = 0; j < NB; ++j) {
      acc[m][j][0] = acc[m][j][1] = acc[m][j][2] = acc[m][j][3] = 0.f;
      if constexpr (GLU) { acu[m][j][0] = acu[m][j][1] = acu[m][j][2] = acu[m][j][3] = 0.f; }
    }
  const int wrow = ROWS >= 64 ? (warp >> 1) * 32 : 0;     // the warp's first row of the tile
  const int wcol = ROWS >= 64 ? (warp & 1) * 32 : warp * 16;   // and first column
  for (int t = 0; t < ksl; ++t) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    if (t + STAGES - 1 < ksl) issue(t + STAGES - 1); else cp_async_commit();
    const uint32_t st = s0 + (t % STAGES) * STAGE;
#pragma unroll
    for (int ks = 0; ks < BK / 16; ++ks) {
      uint32_t af[MB][4];
#pragma unroll
      for (int m = 0; m < MB; ++m)
        ldmatrix_x4(af[m], st + (wrow + m * 16 + (lane & 15)) * SROW * 2 + (ks * 2 + (lane >> 4)) * 16);
#pragma unroll
      for (int jb = 0; jb < NB / 2; ++jb) {
        uint32_t wf[4];
        const int mi = lane >> 3;
        const uint32_t off = (wcol + jb * 16 + (mi >> 1) * 8 + (lane & 7)) * SROW * 2 + (ks * 2 + (mi & 1)) * 16;
        ldmatrix_x4(wf, st + A_BYTES + off);
#pragma unroll
        for (int m = 0; m < MB; ++m) {
          mma_bf16(acc[m][2 * jb], af[m], wf[0], wf[1]);
          mma_bf16(acc[m][2 * jb + 1], af[m], wf[2], wf[3]);
        }
        if constexpr (GLU) {
          ldmatrix_x4(wf, st + A_BYTES + W_BYTES + off);
#pragma unroll
          for (int m = 0; m < MB; ++m) {
            mma_bf16(acu[m][2 * jb], af[m], wf[0], wf[1]);
            mma_bf16(acu[m][2 * jb + 1], af[m], wf[2], wf[3]);
          }
        }
      }
    }
  }
  cp_async_wait<0>();
  TC* C = (TC*)p.C + (p.tiles ? 0 : (long long)group * p.c_group);
#pragma unroll
  for (int mh = 0; mh < 2 * MB; ++mh) {
    const int m = mh >> 1, hh = mh & 1;
    const int cr = crow_s[wrow + m * 16 + (lane >> 2) + 8 * hh];
    if (cr < 0) continue;
#pragma unroll
    for (int j = 0; j < NB; ++j) {
      const int n = n0 + wcol + 8 * j + 2 * (lane & 3);
      if (n >= N) continue;
      float v0 = acc[m][j][2 * hh], v1 = acc[m][j][2 * hh + 1];
      if constexpr (GLU) {
        const float g0 = fminf(v0, p.limit), g1 = fminf(v1, p.limit);
        const float u0 = fminf(fmaxf(acu[m][j][2 * hh], -p.limit), p.limit), u1 = fminf(fmaxf(acu[m][j][2 * hh + 1], -p.limit), p.limit);
        v0 = g0 * (1.0f / (1.0f + expf(-p.alpha * g0))) * (u0 + p.up_shift);
        v1 = g1 * (1.0f / (1.0f + expf(-p.alpha * g1))) * (u1 + p.up_shift);
      }
      store2<TC>(C + (long long)cr * p.ldc + n, v0, v1);
    }
  }
}

template <int ROWS, typename TC, bool GLU>
int launch(const GroupedArgs& p, dim3 grid, cudaStream_t stream) {
  constexpr int SROW = Slice<ROWS>::SROW;
  constexpr size_t smem = (size_t)STAGES * (ROWS * SROW * 2 + (GLU ? 2 : 1) * BN * SROW * 2);
  auto kern = grouped_gemm_tc_kernel<ROWS, TC, GLU>;
  static bool raised = false;
  if (smem > 48 * 1024 && !raised) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    raised = true;
  }
  fz_launch(kern, grid, dim3(ROWS == 128 ? 256 : 128), smem, stream, p);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

template <int ROWS>
int dispatch(const GroupedArgs& p, dim3 grid, int out_dtype, bool glu, cudaStream_t stream) {
  if (out_dtype == FZ_BF16) return glu ? launch<ROWS, __nv_bfloat16, true>(p, grid, stream) : launch<ROWS, __nv_bfloat16, false>(p, grid, stream);
  if (out_dtype == FZ_F32 && !glu) return launch<ROWS, float, false>(p, grid, stream);
  return FZ_BAD_DTYPE;
}

bool aligned16(const void* ptr) { return ((uintptr_t)ptr & 15) == 0; }
}  // namespace

// 0 if the tensor-core kernels take a product with these strides (in elements) and sizes.
FZ_API int fz_grouped_tc_check(const void* A, long long lda, long long a_group, const void* W, const void* C,
                               long long ldc, long long c_group, int N, int K) {
  if (K <= 0 || N <= 0 || K % 8 || N % 2 || lda % 8 || a_group % 8 || ldc % 2 || c_group % 2) return FZ_BAD_SHAPE;
  if (!aligned16(A) || !aligned16(W) || ((uintptr_t)C & 7)) return FZ_BAD_ALIGNMENT;
  return FZ_OK;
}

// One product per head (see fz_linear_heads). rows_per_tile: 16 or 64.
FZ_API int fz_linear_heads_tc(const void* A, long long lda, long long a_head, const void* W, void* C, long long ldc,
                              long long c_head, int out_dtype, int M, int H, int N, int K, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || H <= 0) return FZ_OK;
  if (fz_grouped_tc_check(A, lda, a_head, W, C, ldc, c_head, N, K) != FZ_OK) return FZ_BAD_SHAPE;
  const int rows = M <= 16 ? 16 : M >= 256 ? 128 : 64;
  if (H > 65535 || (M + rows - 1) / rows > 65535) return FZ_TOO_LARGE;
  GroupedArgs p = {(const __nv_bfloat16*)A, lda, a_head, (const __nv_bfloat16*)W, (long long)N * K, C, ldc, c_head, M, N, K,
                   nullptr, nullptr, nullptr, 0.f, 0.f, 0.f, nullptr, 0, 0};
  const dim3 grid((N + BN - 1) / BN, (M + rows - 1) / rows, H);
  return rows == 16 ? dispatch<16>(p, grid, out_dtype, false, stream)
       : rows == 64 ? dispatch<64>(p, grid, out_dtype, false, stream) : dispatch<128>(p, grid, out_dtype, false, stream);
}

// Experts mode (see fz_grouped_linear). tile_rows: the rows per tile the tile list was built for: 16, 64 or 128.
FZ_API int fz_grouped_linear_tc(const void* A, const void* W, void* C, const int* tiles, int max_tiles, int tile_rows,
                                const int* a_idx, const int* c_idx, int out_dtype, int N, int K, int glu, float alpha,
                                float limit, float up_shift, const int* pad_rows, int pad_n, int pad_top, cudaStream_t stream) {
  if (max_tiles <= 0 || N <= 0) return FZ_OK;
  if (fz_grouped_tc_check(A, K, 0, W, C, N, 0, N, K) != FZ_OK || (tile_rows != 16 && tile_rows != 64 && tile_rows != 128)) return FZ_BAD_SHAPE;
  if (max_tiles > 65535) return FZ_TOO_LARGE;
  GroupedArgs p = {(const __nv_bfloat16*)A, K, 0, (const __nv_bfloat16*)W, (long long)(glu ? 2 : 1) * N * K, C, N, 0, 0, N, K,
                   tiles, a_idx, c_idx, alpha, limit, up_shift, pad_rows, pad_n, pad_top};
  const dim3 grid((N + BN - 1) / BN, max_tiles, 1);
  return tile_rows == 16 ? dispatch<16>(p, grid, out_dtype, glu != 0, stream)
       : tile_rows == 64 ? dispatch<64>(p, grid, out_dtype, glu != 0, stream) : dispatch<128>(p, grid, out_dtype, glu != 0, stream);
}

#ifdef FZ_TIMELINE
FZ_TIMELINE_READER(grouped_gemm_tc)
#endif
