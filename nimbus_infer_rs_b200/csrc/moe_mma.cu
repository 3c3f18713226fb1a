// The per-expert products of a routed feed-forward on the tensor cores (bf16 operands, fp32
// accumulation): the same contract as nb_moe_gemm, for bf16 rows and weights with K % 8 == 0.
//
// A CTA takes 64 places of one expert's group and 64 outputs; four warps of 16 places each.
// Rows (gathered through `order`) and weight rows come into shared memory in K-blocks of 64
// by 16-byte asynchronous copies, two blocks in flight, zero-filled beyond the group's end,
// the last output and K; operands are read with ldmatrix.  With a second weight set both
// products share the staged rows and the epilogue writes act(a) * b.  A one-token step has a
// handful of places per expert: the tile is mostly empty then and the kernel is a stream of
// the chosen experts' weights, 64 outputs per CTA.
#include "mma_common.cuh"

namespace {

using namespace nbmma;
typedef __nv_bfloat16 bf16;

constexpr int BM = 64, BN = 64, BK = 64, LD = BK + 8, THREADS = 128, STAGES = 2;

template <bool DUAL, typename TY>
__global__ void __launch_bounds__(THREADS)
moe_mma_kernel(const bf16* x, int x_stride, const int* order, int row_div, const int* offsets,
               int n_experts, const bf16* __restrict__ W, const bf16* __restrict__ W2, TY* y,
               int y_stride, int N, int K, int act) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* As = reinterpret_cast<bf16*>(smem_raw);       // [STAGES][BM][LD]
  bf16* Ws = As + STAGES * BM * LD;                    // [STAGES][BN][LD]
  bf16* Ws2 = Ws + STAGES * BN * LD;                   // [STAGES][BN][LD] when DUAL
  __shared__ int a_row[BM];

  int tile = blockIdx.x, e = 0, begin = 0, end = 0;
  for (; e < n_experts; ++e) {
    begin = offsets[e];
    end = offsets[e + 1];
    const int t = (end - begin + BM - 1) / BM;
    if (tile < t) break;
    tile -= t;
  }
  if (e >= n_experts) return;
  const int m0 = begin + tile * BM, n0 = blockIdx.y * BN;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid < BM) {
    const int p = m0 + tid;
    a_row[tid] = p < end ? (order != nullptr ? order[p] / row_div : p) : -1;
  }
  __syncthreads();
  const bf16* We = W + (size_t)e * N * K;
  const bf16* We2 = DUAL ? W2 + (size_t)e * N * K : nullptr;

  auto load_stage = [&](int stage, int k0) {
    for (int i = tid; i < BM * (BK / 8); i += THREADS) {
      const int rr = i >> 3, k = k0 + (i & 7) * 8;
      const int src = a_row[rr];
      const bool ok = src >= 0 && k < K;
      cp_async16_zfill(As + (stage * BM + rr) * LD + (i & 7) * 8,
                       ok ? x + (size_t)src * x_stride + k : x, ok);
    }
    for (int i = tid; i < BN * (BK / 8); i += THREADS) {
      const int rr = i >> 3, k = k0 + (i & 7) * 8;
      const bool ok = n0 + rr < N && k < K;
      const size_t off = (size_t)(n0 + rr) * K + k;
      cp_async16_zfill(Ws + (stage * BN + rr) * LD + (i & 7) * 8, ok ? We + off : We, ok);
      if (DUAL) cp_async16_zfill(Ws2 + (stage * BN + rr) * LD + (i & 7) * 8, ok ? We2 + off : We2, ok);
    }
  };

  float acc[8][4], acc2[DUAL ? 8 : 1][4];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;
#pragma unroll
  for (int i = 0; i < (DUAL ? 8 : 1); ++i) acc2[i][0] = acc2[i][1] = acc2[i][2] = acc2[i][3] = 0.0f;
  const bool warp_has_rows = m0 + warp * 16 < end;

  const int n_k = (K + BK - 1) / BK;
  load_stage(0, 0);
  cp_async_commit();
  for (int kt = 0; kt < n_k; ++kt) {
    const int stage = kt & 1;
    if (kt + 1 < n_k) load_stage(stage ^ 1, (kt + 1) * BK);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    if (warp_has_rows) {
      const bf16* A = As + stage * BM * LD;
      const bf16* B = Ws + stage * BN * LD;
      const bf16* B2 = Ws2 + stage * BN * LD;
#pragma unroll
      for (int kk = 0; kk < BK / 16; ++kk) {
        uint32_t a[4];
        ldmatrix_x4(a, A + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + kk * 16 +
                           (lane >> 4) * 8);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int off = (j * 16 + (lane >> 4) * 8 + (lane & 7)) * LD + kk * 16 + ((lane >> 3) & 1) * 8;
          uint32_t b[4];
          ldmatrix_x4(b, B + off);
          mma_bf16(acc[2 * j], a, b[0], b[1]);
          mma_bf16(acc[2 * j + 1], a, b[2], b[3]);
          if (DUAL) {
            ldmatrix_x4(b, B2 + off);
            mma_bf16(acc2[2 * j], a, b[0], b[1]);
            mma_bf16(acc2[2 * j + 1], a, b[2], b[3]);
          }
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  if (!warp_has_rows) return;
  const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int p = m0 + warp * 16 + g + half * 8;
    if (p >= end) continue;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int n = n0 + nt * 8 + 2 * t4 + c;
        if (n >= N) continue;
        float v = acc[nt][2 * half + c];
        if (DUAL) v = nb_apply_act_fast(v, act) * acc2[nt][2 * half + c];
        y[(size_t)p * y_stride + n] = nb_from_f32<TY>(v);
      }
    }
  }
}

template <bool DUAL, typename TY>
int launch(dim3 grid, cudaStream_t stream, const bf16* x, int x_stride, const int* order, int row_div,
           const int* offsets, int n_experts, const bf16* W, const bf16* W2, TY* y, int y_stride,
           int N, int K, int act) {
  const size_t smem = (size_t)STAGES * (BM + BN * (DUAL ? 2 : 1)) * LD * sizeof(bf16);
  static bool set = false;
  if (!set) {
    NB_CUDA(cudaFuncSetAttribute(moe_mma_kernel<DUAL, TY>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem));
    set = true;
  }
  NB_CUDA(nb_launch(moe_mma_kernel<DUAL, TY>, grid, dim3(THREADS), smem, stream, x, x_stride, order,
                    row_div, offsets, n_experts, W, W2, y, y_stride, N, K, act));
  return 0;
}

}  // namespace

NB_EXPORT int nb_moe_gemm_mma_supported(int x_dtype, int w_dtype, int x_stride, int K) {
  return x_dtype == NB_BF16 && w_dtype == NB_BF16 && K % 8 == 0 && x_stride % 8 == 0;
}

NB_EXPORT int nb_moe_gemm_mma(const void* x, int x_stride, const int* order, int row_div,
                              const int* offsets, int n_experts, int n_pairs, const void* W,
                              const void* W2, void* y, int y_dtype, int y_stride, int N, int K, int act,
                              cudaStream_t stream) {
  if (n_pairs == 0) return 0;
  NB_REQUIRE(N > 0 && K > 0 && K % 8 == 0 && x_stride % 8 == 0 && n_experts >= 1 && row_div >= 1,
             NB_ERR_BAD_ARG, "moe_gemm_mma: bad sizes N=%d K=%d stride=%d", N, K, x_stride);
  NB_REQUIRE(((uintptr_t)x | (uintptr_t)W | (uintptr_t)W2) % 16 == 0, NB_ERR_BAD_ARG,
             "moe_gemm_mma: pointers must be 16-byte aligned");
  const int tiles = (n_pairs + BM - 1) / BM + (n_experts < n_pairs ? n_experts : n_pairs);
  const dim3 grid(tiles, (N + BN - 1) / BN);
  NB_REQUIRE(grid.y <= 65535, NB_ERR_UNSUPPORTED, "moe_gemm_mma: %d outputs are too many", N);
  int rc;
  const bf16* xb = (const bf16*)x;
  const bf16* w = (const bf16*)W;
  const bf16* w2 = (const bf16*)W2;
  if (y_dtype == NB_BF16) {
    rc = W2 ? launch<true, bf16>(grid, stream, xb, x_stride, order, row_div, offsets, n_experts, w, w2,
                                 (bf16*)y, y_stride, N, K, act)
            : launch<false, bf16>(grid, stream, xb, x_stride, order, row_div, offsets, n_experts, w, w2,
                                  (bf16*)y, y_stride, N, K, act);
  } else if (y_dtype == NB_F32) {
    rc = W2 ? launch<true, float>(grid, stream, xb, x_stride, order, row_div, offsets, n_experts, w, w2,
                                  (float*)y, y_stride, N, K, act)
            : launch<false, float>(grid, stream, xb, x_stride, order, row_div, offsets, n_experts, w, w2,
                                   (float*)y, y_stride, N, K, act);
  } else {
    NB_REQUIRE(false, NB_ERR_BAD_ARG, "moe_gemm_mma: unknown output dtype %d", y_dtype);
  }
  if (rc) return rc;
  NB_CHECK_LAUNCH("moe_gemm_mma");
  return 0;
}
