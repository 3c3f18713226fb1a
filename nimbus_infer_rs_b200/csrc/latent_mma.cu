// Attention over cached latents on the tensor cores (bf16 operands, fp32 accumulation and
// softmax), for prompts and for one-token steps alike.
//
// Every head of a token attends over the same cached rows (a token's latent is its key and
// its value for all heads), so the (token, head) pairs of a sequence are the rows of ONE query
// matrix: a CTA takes 64 consecutive pairs (16 per warp), walks over the pages of 64 cached
// latents that any of its rows may see, and per page computes S = Q C^T (contraction over the
// latent's dims), masks by each row's position (and window), updates the running maximum and
// sum in fp32, and adds P C to the output accumulators (contraction over the page's keys, C
// read through transposing ldmatrix loads from the same shared-memory tile).  Pages come in
// by 16-byte asynchronous copies, two in flight.
//
// When there are too few CTAs to fill the GPU (one-token steps, short prompts) the pages of a
// tile are cut into `n_splits` runs, one CTA each; the runs leave unnormalised sums with their
// maximum and denominator in scratch memory and `latent_merge_kernel` adds them up.  The sink
// (a term of the denominator with no key and no value) enters where the row is finished: in
// the attention kernel without splits, in the merge with.
#include "mma_common.cuh"

namespace {

using namespace nbmma;
typedef __nv_bfloat16 bf16;

constexpr int PAGE_KEYS = 64;
constexpr int TILE = 64;       // (token, head) pairs per CTA
constexpr int THREADS = 128;
constexpr float LOG2E = 1.4426950408889634f;

template <int NT>   // the latent's size rounded up to NT * 16
__global__ void __launch_bounds__(THREADS)
latent_mma_kernel(const bf16* q, const int* cu_rows, const int* seq_slot, const int* seq_pos0,
                  const bf16* cache, const int* block_table, int max_pages, int R, int H,
                  const float* sink, bf16* out, float scale_log2, int window, int n_splits,
                  float* part_o, float* part_ml) {
  constexpr int RP = NT * 16, LD = RP + 8;
  nb_grid_dependency_wait();
  nb_launch_dependents();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);      // [TILE][LD]
  bf16* Cs = Qs + TILE * LD;                          // [2][PAGE_KEYS][LD]

  const int tile = blockIdx.x, s = blockIdx.y, z = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const int row0 = cu_rows[s], n_tok = cu_rows[s + 1] - row0;
  const int n_pairs = n_tok * H;
  const int p0 = tile * TILE;
  if (p0 >= n_pairs) return;
  const int slot = seq_slot[s], pos0 = seq_pos0[s];
  const int seq_end = pos0 + n_tok;                       // keys the sequence has after this step
  const int t_lo = p0 / H, t_hi = (min(n_pairs, p0 + TILE) - 1) / H;
  const int first_key = window > 0 ? max(0, pos0 + t_lo - window + 1) : 0;
  const int pg_lo = first_key / PAGE_KEYS, pg_hi = (pos0 + t_hi) / PAGE_KEYS + 1;
  const int chunk = (pg_hi - pg_lo + n_splits - 1) / n_splits;
  const int my_lo = pg_lo + z * chunk, my_hi = min(pg_hi, my_lo + chunk);
  const int* pages = block_table + (size_t)slot * max_pages;
  const int chunks_per_row = R >> 3;

  if (R != RP) {   // columns beyond the latent's size take part in the products: zeros
    uint4* p = reinterpret_cast<uint4*>(smem_raw);
    const int n16 = (3 * TILE * LD * (int)sizeof(bf16)) >> 4;
    for (int i = tid; i < n16; i += THREADS) p[i] = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();
  }

  auto load_page = [&](int buf, int pg) {
    const bf16* src = cache + (size_t)pages[pg] * PAGE_KEYS * R;
    bf16* dst = Cs + (size_t)buf * PAGE_KEYS * LD;
    for (int i = tid; i < PAGE_KEYS * chunks_per_row; i += THREADS) {
      const int key = i / chunks_per_row, ch = i - key * chunks_per_row;
      cp_async16_zfill(dst + key * LD + ch * 8, src + (size_t)key * R + ch * 8, true);
    }
  };
  {   // the tile's queries: pair p of the sequence is R consecutive numbers
    const bf16* src = q + (size_t)row0 * H * R + (size_t)p0 * R;
    for (int i = tid; i < TILE * chunks_per_row; i += THREADS) {
      const int rr = i / chunks_per_row, ch = i - rr * chunks_per_row;
      const bool ok = p0 + rr < n_pairs;
      cp_async16_zfill(Qs + rr * LD + ch * 8, ok ? src + (size_t)rr * R + ch * 8 : q, ok);
    }
  }
  if (my_lo < my_hi) load_page(0, my_lo);
  cp_async_commit();

  // this thread's two rows: pairs rA and rA + 8 of the sequence
  const int rA = p0 + warp * 16 + g, rB = rA + 8;
  const int posA = rA < n_pairs ? pos0 + rA / H : -1;
  const int posB = rB < n_pairs ? pos0 + rB / H : -1;
  const int lowA = window > 0 ? posA - window + 1 : 0, lowB = window > 0 ? posB - window + 1 : 0;
  const bool warp_has_rows = p0 + warp * 16 < n_pairs;

  float o[2 * NT][4];
#pragma unroll
  for (int i = 0; i < 2 * NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  float mA = -INFINITY, mB = -INFINITY, lA = 0.0f, lB = 0.0f;

  for (int pg = my_lo; pg < my_hi; ++pg) {
    const int buf = (pg - my_lo) & 1;
    if (pg + 1 < my_hi) load_page(buf ^ 1, pg + 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    bf16* C = Cs + (size_t)buf * PAGE_KEYS * LD;
    const int key0 = pg * PAGE_KEYS;
    if (key0 + PAGE_KEYS > seq_end) {
      // rows of the page that no token of the sequence has written yet: whatever an earlier
      // owner of the page left there must not reach the products (0 x NaN)
      const int first = max(0, seq_end - key0);
      for (int i = tid; i < (PAGE_KEYS - first) * (LD / 8); i += THREADS) {
        const int key = first + i / (LD / 8), ch = i % (LD / 8);
        *reinterpret_cast<uint4*>(C + key * LD + ch * 8) = make_uint4(0u, 0u, 0u, 0u);
      }
      __syncthreads();
    }
    if (warp_has_rows) {
      // S = Q C^T for 16 rows x 64 keys
      float sc[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.0f;
#pragma unroll
      for (int kk = 0; kk < NT; ++kk) {
        uint32_t a[4];
        ldmatrix_x4(a, Qs + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + kk * 16 +
                           (lane >> 4) * 8);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t b[4];
          ldmatrix_x4(b, C + (j * 16 + (lane >> 4) * 8 + (lane & 7)) * LD + kk * 16 +
                             ((lane >> 3) & 1) * 8);
          mma_bf16(sc[2 * j], a, b[0], b[1]);
          mma_bf16(sc[2 * j + 1], a, b[2], b[3]);
        }
      }
      // scale, mask, running maximum
      float mxA = -INFINITY, mxB = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int j = key0 + nt * 8 + 2 * t4 + c;
          float vA = sc[nt][c] * scale_log2, vB = sc[nt][2 + c] * scale_log2;
          if (j > posA || j < lowA) vA = -INFINITY;
          if (j > posB || j < lowB) vB = -INFINITY;
          sc[nt][c] = vA;
          sc[nt][2 + c] = vB;
          mxA = fmaxf(mxA, vA);
          mxB = fmaxf(mxB, vB);
        }
      }
      mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1));
      mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2));
      mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1));
      mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2));
      const float nA = fmaxf(mA, mxA), nB = fmaxf(mB, mxB);
      const float baseA = nA == -INFINITY ? 0.0f : nA, baseB = nB == -INFINITY ? 0.0f : nB;
      const float fA = exp2_fast(mA - baseA), fB = exp2_fast(mB - baseB);   // 0 when m was -inf
      mA = nA;
      mB = nB;
      lA *= fA;
      lB *= fB;
#pragma unroll
      for (int i = 0; i < 2 * NT; ++i) {
        o[i][0] *= fA; o[i][1] *= fA; o[i][2] *= fB; o[i][3] *= fB;
      }
      uint32_t pa[4][4];     // P as the A operand of four k-steps of 16 keys
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const float e0 = exp2_fast(sc[nt][0] - baseA), e1 = exp2_fast(sc[nt][1] - baseA);
        const float e2 = exp2_fast(sc[nt][2] - baseB), e3 = exp2_fast(sc[nt][3] - baseB);
        lA += e0 + e1;
        lB += e2 + e3;
        pa[nt >> 1][(nt & 1) * 2] = pack_bf16(e0, e1);
        pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(e2, e3);
      }
      // O += P C
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, C + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LD + j * 16 +
                                   (lane >> 4) * 8);
          mma_bf16(o[2 * j], pa[kk], b[0], b[1]);
          mma_bf16(o[2 * j + 1], pa[kk], b[2], b[3]);
        }
      }
    }
    __syncthreads();    // the buffer is filled again two pages on
  }
  cp_async_wait<0>();
  if (!warp_has_rows) return;

  lA += __shfl_xor_sync(0xffffffffu, lA, 1);
  lA += __shfl_xor_sync(0xffffffffu, lA, 2);
  lB += __shfl_xor_sync(0xffffffffu, lB, 1);
  lB += __shfl_xor_sync(0xffffffffu, lB, 2);

#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = half ? rB : rA;
    if (r >= n_pairs) continue;
    float m = half ? mB : mA, l = half ? lB : lA;
    const int tok = r / H, h = r - tok * H;
    const size_t pair = (size_t)(row0 + tok) * H + h;
    if (n_splits > 1) {
      float* po = part_o + (pair * n_splits + z) * R;
#pragma unroll
      for (int i = 0; i < 2 * NT; ++i) {
        const int col = i * 8 + 2 * t4;
        if (col < R) *reinterpret_cast<float2*>(po + col) = make_float2(o[i][2 * half], o[i][2 * half + 1]);
      }
      if (t4 == 0) *reinterpret_cast<float2*>(part_ml + (pair * n_splits + z) * 2) = make_float2(m, l);
    } else {
      float f = 1.0f;
      if (sink != nullptr) {
        const float s2 = sink[h] * LOG2E;
        const float mf = fmaxf(m, s2);
        f = exp2_fast(m - mf);
        l = l * f + exp2_fast(s2 - mf);
      }
      const float inv = l > 0.0f ? f / l : 0.0f;
      bf16* dst = out + pair * R;
#pragma unroll
      for (int i = 0; i < 2 * NT; ++i) {
        const int col = i * 8 + 2 * t4;
        if (col < R)
          *reinterpret_cast<uint32_t*>(dst + col) = pack_bf16(o[i][2 * half] * inv, o[i][2 * half + 1] * inv);
      }
    }
  }
}

// One CTA per (row, head): add up the runs of a split launch, put the sink into the
// denominator, write the result.  Maxima are in units of log2.
__global__ void latent_merge_kernel(const float* part_o, const float* part_ml, const int* row_slot,
                                    const float* sink, bf16* out, int H, int R, int n_splits) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  const size_t pair = blockIdx.x;
  const int row = (int)(pair / H), h = (int)(pair % H);
  bf16* dst = out + pair * R;
  if (row_slot[row] < 0) {
    for (int d = threadIdx.x; d < R; d += blockDim.x) dst[d] = __float2bfloat16_rn(0.0f);
    return;
  }
  const float* ml = part_ml + pair * n_splits * 2;
  float m = sink != nullptr ? sink[h] * LOG2E : -INFINITY;
  for (int i = 0; i < n_splits; ++i)
    if (ml[2 * i + 1] > 0.0f) m = fmaxf(m, ml[2 * i]);
  float l = sink != nullptr ? exp2_fast(sink[h] * LOG2E - m) : 0.0f;
  for (int i = 0; i < n_splits; ++i)
    if (ml[2 * i + 1] > 0.0f) l += ml[2 * i + 1] * exp2_fast(ml[2 * i] - m);
  const float inv = l > 0.0f ? 1.0f / l : 0.0f;
  for (int d = threadIdx.x; d < R; d += blockDim.x) {
    float acc = 0.0f;
    for (int i = 0; i < n_splits; ++i)
      if (ml[2 * i + 1] > 0.0f)
        acc = fmaf(part_o[(pair * n_splits + i) * R + d], exp2_fast(ml[2 * i] - m), acc);
    dst[d] = __float2bfloat16_rn(acc * inv);
  }
}

template <int NT>
int launch(const bf16* q, const int* cu_rows, const int* seq_slot, const int* seq_pos0,
           const bf16* cache, const int* block_table, int max_pages, int R, int H, const float* sink,
           bf16* out, float scale, int window, int n_seqs, int max_q_len, int n_splits,
           float* part_o, float* part_ml, cudaStream_t stream) {
  constexpr int LD = NT * 16 + 8;
  const size_t smem = (size_t)3 * TILE * LD * sizeof(bf16);
  static bool set = false;
  if (!set) {
    NB_CUDA(cudaFuncSetAttribute(latent_mma_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem));
    set = true;
  }
  const dim3 grid(((size_t)max_q_len * H + TILE - 1) / TILE, n_seqs, n_splits);
  NB_CUDA(nb_launch(latent_mma_kernel<NT>, grid, dim3(THREADS), smem, stream, q, cu_rows, seq_slot,
                    seq_pos0, cache, block_table, max_pages, R, H, sink, out, scale * LOG2E, window,
                    n_splits, part_o, part_ml));
  return 0;
}

}  // namespace

// Whether the tensor-core kernel takes this shape (else the caller uses nb_attention_latent).
NB_EXPORT int nb_attention_latent_mma_supported(int rank, int page, int n_heads) {
  return rank % 8 == 0 && rank >= 8 && rank <= 256 && page == PAGE_KEYS && n_heads >= 1;
}

// q, out: bf16 [n_rows][n_heads * rank], contiguous; cache: bf16 one plane [n_pages][64][rank];
// part_o / part_ml: fp32 scratch of n_rows * n_heads * n_splits * rank and ... * 2 numbers
// (needed when n_splits > 1).  max_q_len: the longest run of rows of one sequence.
NB_EXPORT int nb_attention_latent_mma(const void* q, const int* cu_rows, const int* seq_slot,
                                      const int* seq_pos0, const int* row_slot, const void* cache,
                                      const int* block_table, int max_pages, int page, int n_heads,
                                      int rank, const float* sink, void* out, float scale, int window,
                                      int n_rows, int n_seqs, int max_q_len, int n_splits,
                                      float* part_o, float* part_ml, cudaStream_t stream) {
  if (n_rows == 0 || n_seqs == 0) return 0;
  NB_REQUIRE(nb_attention_latent_mma_supported(rank, page, n_heads), NB_ERR_UNSUPPORTED,
             "attention_latent_mma: latent size %d / page %d not supported", rank, page);
  NB_REQUIRE(n_splits >= 1 && n_splits <= 64 && (n_splits == 1 || (part_o && part_ml)), NB_ERR_BAD_ARG,
             "attention_latent_mma: bad splits %d", n_splits);
  NB_REQUIRE(((uintptr_t)q | (uintptr_t)cache | (uintptr_t)out) % 16 == 0, NB_ERR_BAD_ARG,
             "attention_latent_mma: pointers must be 16-byte aligned");
  NB_REQUIRE(n_seqs <= 65535, NB_ERR_UNSUPPORTED, "attention_latent_mma: too many sequences");
  const int nt = (rank + 15) / 16;
  int rc;
#define NB_LM(N_)                                                                                  \
  rc = launch<N_>((const bf16*)q, cu_rows, seq_slot, seq_pos0, (const bf16*)cache, block_table,    \
                  max_pages, rank, n_heads, sink, (bf16*)out, scale, window, n_seqs, max_q_len,    \
                  n_splits, part_o, part_ml, stream)
  if (nt <= 2) NB_LM(2);
  else if (nt <= 4) NB_LM(4);
  else if (nt <= 6) NB_LM(6);
  else if (nt <= 8) NB_LM(8);
  else if (nt <= 12) NB_LM(12);
  else NB_LM(16);
#undef NB_LM
  if (rc) return rc;
  NB_CHECK_LAUNCH("attention_latent_mma");
  if (n_splits > 1) {
    NB_CUDA(nb_launch(latent_merge_kernel, dim3((unsigned)((size_t)n_rows * n_heads)), dim3(64), 0, stream,
                      (const float*)part_o, (const float*)part_ml, row_slot, sink, (bf16*)out, n_heads,
                      rank, n_splits));
    NB_CHECK_LAUNCH("latent_merge");
  }
  return 0;
}
