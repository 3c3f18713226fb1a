// Products per group of rows on the tensor cores (bf16 operands, fp32 accumulation): the
// per-expert products of a routed feed-forward (the contract of nb_moe_gemm, for bf16 rows and
// weights with K % 8 == 0; a group = the places of one expert), and the per-head linear maps of
// the latent attention (the contract of nb_head_linear; a group = one head, every row of the
// step belongs to every group, each group reads and writes its own columns).
//
// A CTA takes 128 places of one group and 64 outputs; eight warps, each 32 places x 32
// outputs (two by four MMA tiles, so an operand fetched from shared memory feeds several
// MMAs).  Rows (gathered through `order`) and weight rows come into shared memory in K-blocks
// of 64 by 16-byte asynchronous copies through a ring of three stages, zero-filled beyond the
// group's end, the last output and K; operands are read with ldmatrix.  With a second weight
// set both products share the staged rows and the epilogue writes act(a) * b.  A one-token
// step has a handful of places per expert: the tile is mostly empty then (warps without rows
// skip the MMAs) and the kernel is a stream of the chosen experts' weights, 64 outputs per CTA.
#include "mma_common.cuh"

namespace {

using namespace nbmma;
typedef __nv_bfloat16 bf16;

constexpr int BM = 128, BN = 64, BK = 64, LD = BK + 8, THREADS = 256, STAGES = 3;

// Groups are either given by `offsets` (group e = places offsets[e] .. offsets[e+1]; a place's
// source row is order[place] / row_div, or the place itself) or, with `uniform_rows` > 0, every
// group has rows 0 .. uniform_rows - 1, reads columns e * x_gcol .. of x and writes columns
// e * y_gcol .. of y; rows with a negative `row_slot` then give zeros, and with `gate` the
// result is multiplied by sigmoid(gate[row][gate_col + e]).
template <bool DUAL, typename TX, typename TY>
__global__ void __launch_bounds__(THREADS)
moe_mma_kernel(const TX* x, int x_stride, const int* order, int row_div, const int* offsets,
               int n_experts, const bf16* __restrict__ W, const bf16* __restrict__ W2, TY* y,
               int y_stride, int N, int K, int act, int uniform_rows, int x_gcol, int y_gcol,
               const int* row_slot, const float* gate, int gate_stride, int gate_col) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* As = reinterpret_cast<bf16*>(smem_raw);       // [STAGES][BM][LD]
  bf16* Ws = As + STAGES * BM * LD;                    // [STAGES][BN][LD]
  bf16* Ws2 = Ws + STAGES * BN * LD;                   // [STAGES][BN][LD] when DUAL
  __shared__ int a_row[BM];

  int tile = blockIdx.x, e = 0, begin = 0, end = 0;
  if (uniform_rows > 0) {
    const int per = (uniform_rows + BM - 1) / BM;
    e = tile / per;
    tile -= e * per;
    end = uniform_rows;
  } else {
    for (; e < n_experts; ++e) {
      begin = offsets[e];
      end = offsets[e + 1];
      const int t = (end - begin + BM - 1) / BM;
      if (tile < t) break;
      tile -= t;
    }
  }
  if (e >= n_experts) return;
  const int m0 = begin + tile * BM, n0 = blockIdx.y * BN;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid < BM) {
    const int p = m0 + tid;
    int src = p < end ? (order != nullptr ? order[p] / row_div : p) : -1;
    if (src >= 0 && uniform_rows > 0 && row_slot[src] < 0) src = -1;
    a_row[tid] = src;
  }
  __syncthreads();
  x += (size_t)e * x_gcol;
  y += (size_t)e * y_gcol;
  // 32-bit rows can be fetched 16 bytes at a time when every row's piece starts on such a boundary
  const bool x_vec4 = sizeof(TX) == 4 && x_stride % 4 == 0 && x_gcol % 4 == 0 &&
                      (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  const bf16* We = W + (size_t)e * N * K;
  const bf16* We2 = DUAL ? W2 + (size_t)e * N * K : nullptr;

  auto load_stage = [&](int stage, int k0) {
    if constexpr (sizeof(TX) == 2) {
      for (int i = tid; i < BM * (BK / 8); i += THREADS) {
        const int rr = i >> 3, k = k0 + (i & 7) * 8;
        const int src = a_row[rr];
        const bool ok = src >= 0 && k < K;
        cp_async16_zfill(As + (stage * BM + rr) * LD + (i & 7) * 8,
                         ok ? x + (size_t)src * x_stride + k : x, ok);
      }
    } else if (x_vec4) {   // 32-bit rows: rounded to bf16 on the way into shared memory
      constexpr int PER = BM * BK / 4 / THREADS;
      float4 v[PER];
#pragma unroll
      for (int u = 0; u < PER; ++u) {      // all loads first, then the stores
        const int i = tid + u * THREADS, rr = i / (BK / 4), k = k0 + (i % (BK / 4)) * 4;
        const int src = a_row[rr];
        v[u] = (src >= 0 && k < K)
                   ? *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + (size_t)src * x_stride + k)
                   : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      }
#pragma unroll
      for (int u = 0; u < PER; ++u) {
        const int i = tid + u * THREADS, rr = i / (BK / 4), kk = (i % (BK / 4)) * 4;
        uint2 pk;
        pk.x = pack_bf16(v[u].x, v[u].y);
        pk.y = pack_bf16(v[u].z, v[u].w);
        *reinterpret_cast<uint2*>(As + (stage * BM + rr) * LD + kk) = pk;
      }
    } else {
      for (int i = tid; i < BM * BK; i += THREADS) {
        const int rr = i / BK, kk = i % BK;
        const int src = a_row[rr];
        const float v = (src >= 0 && k0 + kk < K) ? nb_to_f32(x[(size_t)src * x_stride + k0 + kk]) : 0.0f;
        As[(stage * BM + rr) * LD + kk] = __float2bfloat16_rn(v);
      }
    }
    for (int i = tid; i < BN * (BK / 8); i += THREADS) {
      const int rr = i >> 3, k = k0 + (i & 7) * 8;
      const bool ok = n0 + rr < N && k < K;
      const size_t off = (size_t)(n0 + rr) * K + k;
      cp_async16_zfill(Ws + (stage * BN + rr) * LD + (i & 7) * 8, ok ? We + off : We, ok);
      if (DUAL) cp_async16_zfill(Ws2 + (stage * BN + rr) * LD + (i & 7) * 8, ok ? We2 + off : We2, ok);
    }
  };

  const int wm = warp >> 1, wn = warp & 1;      // the warp's 32 places and 32 outputs
  float acc[2][4][4], acc2[DUAL ? 2 : 1][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.0f;
#pragma unroll
  for (int i = 0; i < (DUAL ? 2 : 1); ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc2[i][j][0] = acc2[i][j][1] = acc2[i][j][2] = acc2[i][j][3] = 0.0f;
  const bool warp_has_rows = m0 + wm * 32 < end;

  const int n_k = (K + BK - 1) / BK;
  load_stage(0, 0);
  cp_async_commit();
  if (n_k > 1) load_stage(1, BK);
  cp_async_commit();
  for (int kt = 0; kt < n_k; ++kt) {
    const int stage = kt % STAGES;
    cp_async_wait<1>();
    __syncthreads();          // block kt has landed, and every warp is done with block kt - 1
    if (kt + 2 < n_k) load_stage((kt + 2) % STAGES, (kt + 2) * BK);
    cp_async_commit();
    if (warp_has_rows) {
      const bf16* A = As + stage * BM * LD;
      const bf16* B = Ws + stage * BN * LD;
      const bf16* B2 = Ws2 + stage * BN * LD;
#pragma unroll
      for (int kk = 0; kk < BK / 16; ++kk) {
        uint32_t a[2][4];
#pragma unroll
        for (int mi = 0; mi < 2; ++mi)
          ldmatrix_x4(a[mi], A + (wm * 32 + mi * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD +
                                 kk * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int off = (wn * 32 + j * 16 + (lane >> 4) * 8 + (lane & 7)) * LD + kk * 16 +
                          ((lane >> 3) & 1) * 8;
          uint32_t b[4];
          ldmatrix_x4(b, B + off);
#pragma unroll
          for (int mi = 0; mi < 2; ++mi) {
            mma_bf16(acc[mi][2 * j], a[mi], b[0], b[1]);
            mma_bf16(acc[mi][2 * j + 1], a[mi], b[2], b[3]);
          }
          if (DUAL) {
            ldmatrix_x4(b, B2 + off);
#pragma unroll
            for (int mi = 0; mi < 2; ++mi) {
              mma_bf16(acc2[mi][2 * j], a[mi], b[0], b[1]);
              mma_bf16(acc2[mi][2 * j + 1], a[mi], b[2], b[3]);
            }
          }
        }
      }
    }
  }
  cp_async_wait<0>();
  if (!warp_has_rows) return;
  const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
  for (int mi = 0; mi < 2; ++mi) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int local = wm * 32 + mi * 16 + g + half * 8;
      const int p = m0 + local;
      if (p >= end) continue;
      float scale = 1.0f;
      if (uniform_rows > 0) {
        if (a_row[local] < 0) scale = 0.0f;
        else if (gate != nullptr) scale = nb_sigmoid(gate[(size_t)p * gate_stride + gate_col + e]);
      }
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int n = n0 + wn * 32 + nt * 8 + 2 * t4 + c;
          if (n >= N) continue;
          float v = acc[mi][nt][2 * half + c];
          if (DUAL) v = nb_apply_act_fast(v, act) * acc2[mi][nt][2 * half + c];
          y[(size_t)p * y_stride + n] = nb_from_f32<TY>(scale == 0.0f ? 0.0f : v * scale);
        }
      }
    }
  }
}

struct Uniform {      // the per-head form (see the kernel)
  int rows = 0, x_gcol = 0, y_gcol = 0;
  const int* row_slot = nullptr;
  const float* gate = nullptr;
  int gate_stride = 0, gate_col = 0;
};

template <bool DUAL, typename TX, typename TY>
int launch(dim3 grid, cudaStream_t stream, const TX* x, int x_stride, const int* order, int row_div,
           const int* offsets, int n_experts, const bf16* W, const bf16* W2, TY* y, int y_stride,
           int N, int K, int act, Uniform u = Uniform()) {
  const size_t smem = (size_t)STAGES * (BM + BN * (DUAL ? 2 : 1)) * LD * sizeof(bf16);
  static bool set = false;
  if (!set) {
    NB_CUDA(cudaFuncSetAttribute(moe_mma_kernel<DUAL, TX, TY>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    set = true;
  }
  NB_CUDA(nb_launch(moe_mma_kernel<DUAL, TX, TY>, grid, dim3(THREADS), smem, stream, x, x_stride, order,
                    row_div, offsets, n_experts, W, W2, y, y_stride, N, K, act, u.rows, u.x_gcol,
                    u.y_gcol, u.row_slot, u.gate, u.gate_stride, u.gate_col));
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
    rc = W2 ? launch<true, bf16, bf16>(grid, stream, xb, x_stride, order, row_div, offsets, n_experts, w, w2,
                                 (bf16*)y, y_stride, N, K, act)
            : launch<false, bf16, bf16>(grid, stream, xb, x_stride, order, row_div, offsets, n_experts, w, w2,
                                  (bf16*)y, y_stride, N, K, act);
  } else if (y_dtype == NB_F32) {
    rc = W2 ? launch<true, bf16, float>(grid, stream, xb, x_stride, order, row_div, offsets, n_experts, w, w2,
                                  (float*)y, y_stride, N, K, act)
            : launch<false, bf16, float>(grid, stream, xb, x_stride, order, row_div, offsets, n_experts, w, w2,
                                   (float*)y, y_stride, N, K, act);
  } else {
    NB_REQUIRE(false, NB_ERR_BAD_ARG, "moe_gemm_mma: unknown output dtype %d", y_dtype);
  }
  if (rc) return rc;
  NB_CHECK_LAUNCH("moe_gemm_mma");
  return 0;
}

// The per-head linear map (the contract of nb_head_linear) for bf16 weights and bf16 results;
// x: bf16 or fp32 rows (fp32 is rounded to bf16 on the way in).
NB_EXPORT int nb_head_linear_mma_supported(int x_dtype, int w_dtype, int y_dtype, int x_stride,
                                           int x_col, int n_in) {
  return w_dtype == NB_BF16 && y_dtype == NB_BF16 && n_in % 8 == 0 &&
         (x_dtype == NB_F32 || (x_dtype == NB_BF16 && x_stride % 8 == 0 && x_col % 8 == 0));
}

NB_EXPORT int nb_head_linear_mma(const void* x, int x_dtype, int x_stride, int x_col, const void* W,
                                 void* y, int y_stride, const float* gate, int gate_stride,
                                 int gate_col, const int* row_slot, int n_rows, int n_heads, int n_in,
                                 int n_out, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(nb_head_linear_mma_supported(x_dtype, NB_BF16, NB_BF16, x_stride, x_col, n_in),
             NB_ERR_UNSUPPORTED, "head_linear_mma: shape not supported (in=%d stride=%d col=%d)", n_in,
             x_stride, x_col);
  NB_REQUIRE((uintptr_t)W % 16 == 0 && (x_dtype == NB_F32 || (uintptr_t)x % 16 == 0), NB_ERR_BAD_ARG,
             "head_linear_mma: pointers must be 16-byte aligned");
  const dim3 grid((unsigned)(((n_rows + BM - 1) / BM) * n_heads), (n_out + BN - 1) / BN);
  NB_REQUIRE(grid.y <= 65535, NB_ERR_UNSUPPORTED, "head_linear_mma: %d outputs are too many", n_out);
  Uniform u;
  u.rows = n_rows; u.x_gcol = n_in; u.y_gcol = n_out; u.row_slot = row_slot;
  u.gate = gate; u.gate_stride = gate_stride; u.gate_col = gate_col;
  int rc;
  if (x_dtype == NB_F32)
    rc = launch<false, float, bf16>(grid, stream, (const float*)x + x_col, x_stride, nullptr, 1, nullptr,
                                    n_heads, (const bf16*)W, nullptr, (bf16*)y, y_stride, n_out, n_in, 0, u);
  else
    rc = launch<false, bf16, bf16>(grid, stream, (const bf16*)x + x_col, x_stride, nullptr, 1, nullptr,
                                   n_heads, (const bf16*)W, nullptr, (bf16*)y, y_stride, n_out, n_in, 0, u);
  if (rc) return rc;
  NB_CHECK_LAUNCH("head_linear_mma");
  return 0;
}
