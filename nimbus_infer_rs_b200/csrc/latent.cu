// Attention over a cached low-rank latent (one vector of `rank` numbers per token, shared
// by all heads), in fp32 arithmetic on the CUDA cores.
//
// A token's keys and values are linear maps of its latent c: k_h = Wk_h c, v_h = Wv_h c.
// Because the maps are per head and the latent is shared, the maps move to the query side:
//   q_h . k_h(j)      = (Wk_h^T q_h) . c_j
//   sum_j p_j v_h(j)  = Wv_h (sum_j p_j c_j)
// so a step computes a = Wk_h^T q_h per (row, head) once (`nb_head_linear`), attends over the
// cached latents with a as the query and c as key and value at once (`nb_attention_latent`:
// every head reads the same rows), and maps the result through Wv_h (`nb_head_linear` again,
// which also applies a per-head output gate).  Only c is cached: one plane of the paged
// store, written by `nb_latent_append` from the fp32 result of the down projection, normed
// (root mean square, fp32) on the way.
//
// The softmax may have a sink: one more term exp(sink_h) in the denominator that belongs to
// no key and carries no value.
//
// These kernels take any sizes; they are the 32-bit path and what the bf16 path falls back
// to for shapes its tensor-core kernel leaves out.
#include "common.cuh"

namespace {

constexpr int THREADS = 256;
constexpr int CHUNK = 1024;   // keys whose scores are held in shared memory at a time
constexpr int MAX_ACC = 4;    // a thread's dims of the result: rank <= MAX_ACC * THREADS

// ---------------------------------------------------------------------------------
// c = rms(src[r, col : col + rank]) * gamma -> token pos[r] of sequence slot[r] in the
// one-plane paged store [n_pages][1][page][rank].
// ---------------------------------------------------------------------------------
template <typename TC>
__global__ void latent_append_kernel(const float* src, int src_stride, int col,
                                     const float* __restrict__ gamma, float eps,
                                     const int* row_slot, const int* row_pos, TC* cache,
                                     const int* block_table, int max_pages, int page, int rank) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  __shared__ float red[32];
  const int r = blockIdx.x;
  const int slot = row_slot[r];
  if (slot < 0) return;
  const int pos = row_pos[r];
  const float* xr = src + (size_t)r * src_stride + col;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    const float v = xr[i];
    ss = fmaf(v, v, ss);
  }
  ss = nb_block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)rank + eps);
  const int page_id = block_table[(size_t)slot * max_pages + pos / page];
  TC* dst = cache + ((size_t)page_id * page + (pos % page)) * rank;
  for (int i = threadIdx.x; i < rank; i += blockDim.x)
    dst[i] = nb_from_f32<TC>(xr[i] * inv * (gamma ? gamma[i] : 1.0f));
}

// ---------------------------------------------------------------------------------
// y[r, h, o] = g(r, h) * sum_i W[h, o, i] * x[r, x_col + h * n_in + i]
// g = sigmoid(gate[r, gate_col + h]) if `gate` is given, else 1.  A CTA takes ROWS rows of one
// head; each warp walks over outputs, its lanes over the inputs.
// ---------------------------------------------------------------------------------
constexpr int HL_ROWS = 8;

template <typename TX, typename TW, typename TY>
__global__ void __launch_bounds__(THREADS)
head_linear_kernel(const TX* x, int x_stride, int x_col, const TW* __restrict__ W, TY* y,
                   int y_stride, const float* gate, int gate_stride, int gate_col,
                   const int* row_slot, int n_rows, int n_in, int n_out) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  extern __shared__ float xs[];            // [HL_ROWS][n_in]
  const int r0 = blockIdx.x * HL_ROWS, h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nr = min(HL_ROWS, n_rows - r0);
  for (int i = threadIdx.x; i < HL_ROWS * n_in; i += THREADS) {
    const int rr = i / n_in, k = i - rr * n_in;
    float v = 0.0f;
    if (rr < nr && row_slot[r0 + rr] >= 0)
      v = nb_to_f32(x[(size_t)(r0 + rr) * x_stride + x_col + (size_t)h * n_in + k]);
    xs[i] = v;
  }
  __syncthreads();
  const TW* Wh = W + (size_t)h * n_out * n_in;
  for (int o = warp; o < n_out; o += THREADS / 32) {
    float acc[HL_ROWS];
#pragma unroll
    for (int rr = 0; rr < HL_ROWS; ++rr) acc[rr] = 0.0f;
    const TW* wr = Wh + (size_t)o * n_in;
    for (int k = lane; k < n_in; k += 32) {
      const float w = nb_to_f32(wr[k]);
#pragma unroll
      for (int rr = 0; rr < HL_ROWS; ++rr) acc[rr] = fmaf(w, xs[rr * n_in + k], acc[rr]);
    }
#pragma unroll
    for (int rr = 0; rr < HL_ROWS; ++rr) acc[rr] = nb_warp_sum(acc[rr]);
    if (lane < nr) {
      float v = 0.0f;
#pragma unroll
      for (int rr = 0; rr < HL_ROWS; ++rr)
        if (rr == lane) v = acc[rr];
      if (gate != nullptr && row_slot[r0 + lane] >= 0)
        v *= nb_sigmoid(gate[(size_t)(r0 + lane) * gate_stride + gate_col + h]);
      y[(size_t)(r0 + lane) * y_stride + (size_t)h * n_out + o] = nb_from_f32<TY>(v);
    }
  }
}

// ---------------------------------------------------------------------------------
// out[r, h, :] = sum_{j <= pos[r]} p_j c_j,  p_j = exp(s_j) / (sum_j exp(s_j) + exp(sink_h)),
// s_j = scale * a[r, h, :] . c_j.   One CTA per (row, head); warps walk over keys for the
// scores (lanes over the latent's dims), threads over dims for the weighted sum.
// ---------------------------------------------------------------------------------
template <typename TQ, typename TC, typename TOut>
__global__ void __launch_bounds__(THREADS)
attention_latent_kernel(const TQ* q, int q_stride, int q_col, const int* row_slot,
                        const int* row_pos, const TC* cache, const int* block_table,
                        int max_pages, int page, int rank, const float* sink, TOut* out,
                        int out_stride, float scale, int window) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  extern __shared__ float smem[];
  float* q_s = smem;               // [rank]
  float* scores = q_s + rank;      // [CHUNK]
  __shared__ float red[32];

  const int r = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  TOut* o = out + (size_t)r * out_stride + (size_t)h * rank;
  const int slot = row_slot[r];
  if (slot < 0) {
    for (int i = tid; i < rank; i += THREADS) o[i] = nb_from_f32<TOut>(0.0f);
    return;
  }
  const int pos = row_pos[r];
  const int j_begin = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
  const int j_end = pos + 1;
  const int* pages = block_table + (size_t)slot * max_pages;

  const TQ* qr = q + (size_t)r * q_stride + q_col + (size_t)h * rank;
  for (int i = tid; i < rank; i += THREADS) q_s[i] = nb_to_f32(qr[i]);
  __syncthreads();

  float m_run = -INFINITY, l_run = 0.0f;
  float acc[MAX_ACC];
#pragma unroll
  for (int a = 0; a < MAX_ACC; ++a) acc[a] = 0.0f;

  for (int c0 = j_begin; c0 < j_end; c0 += CHUNK) {
    const int c1 = min(c0 + CHUNK, j_end);
    float cmax = -INFINITY;
    for (int j = c0 + warp; j < c1; j += THREADS / 32) {
      const TC* cr = cache + ((size_t)pages[j / page] * page + (j % page)) * rank;
      float dot = 0.0f;
      for (int i = lane; i < rank; i += 32) dot = fmaf(q_s[i], nb_to_f32(cr[i]), dot);
      dot = nb_warp_sum(dot) * scale;
      if (lane == 0) scores[j - c0] = dot;
      cmax = fmaxf(cmax, dot);
    }
    cmax = nb_block_max(cmax, red);
    const float m_new = fmaxf(m_run, cmax);
    float csum = 0.0f;
    for (int j = c0 + tid; j < c1; j += THREADS) {
      const float p = expf(scores[j - c0] - m_new);
      scores[j - c0] = p;
      csum += p;
    }
    csum = nb_block_sum(csum, red);   // also orders the writes of `scores` before the reads below
    const float rescale = (m_run == -INFINITY) ? 0.0f : expf(m_run - m_new);
    l_run = l_run * rescale + csum;
#pragma unroll
    for (int a = 0; a < MAX_ACC; ++a) acc[a] *= rescale;
    for (int j = c0; j < c1; ++j) {
      const TC* cr = cache + ((size_t)pages[j / page] * page + (j % page)) * rank;
      const float p = scores[j - c0];
#pragma unroll
      for (int a = 0; a < MAX_ACC; ++a) {
        const int d = tid + a * THREADS;
        if (d < rank) acc[a] = fmaf(p, nb_to_f32(cr[d]), acc[a]);
      }
    }
    m_run = m_new;
    __syncthreads();   // `scores` is rewritten by the next chunk
  }
  if (sink != nullptr) {
    // one more term of the denominator, with no key and no value
    const float s = sink[h];
    const float m_f = fmaxf(m_run, s);
    const float rescale = expf(m_run - m_f);
    l_run = l_run * rescale + expf(s - m_f);
#pragma unroll
    for (int a = 0; a < MAX_ACC; ++a) acc[a] *= rescale;
  }
  const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
#pragma unroll
  for (int a = 0; a < MAX_ACC; ++a) {
    const int d = tid + a * THREADS;
    if (d < rank) o[d] = nb_from_f32<TOut>(acc[a] * inv);
  }
}

}  // namespace

typedef __nv_bfloat16 bf16;

NB_EXPORT int nb_latent_append(const float* src, int src_stride, int col, const float* gamma,
                               float eps, const int* row_slot, const int* row_pos, void* cache,
                               int cache_dtype, const int* block_table, int max_pages, int page,
                               int rank, int n_rows, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(rank > 0 && col >= 0 && src_stride >= col + rank && page > 0, NB_ERR_BAD_ARG,
             "latent_append: bad sizes rank=%d col=%d stride=%d page=%d", rank, col, src_stride, page);
  const int threads = rank >= 512 ? 256 : (rank >= 128 ? 128 : 64);
  if (cache_dtype == NB_F32)
    NB_CUDA(nb_launch(latent_append_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, src,
                      src_stride, col, gamma, eps, row_slot, row_pos, (float*)cache, block_table,
                      max_pages, page, rank));
  else if (cache_dtype == NB_BF16)
    NB_CUDA(nb_launch(latent_append_kernel<bf16>, dim3(n_rows), dim3(threads), 0, stream, src,
                      src_stride, col, gamma, eps, row_slot, row_pos, (bf16*)cache, block_table,
                      max_pages, page, rank));
  else
    NB_REQUIRE(false, NB_ERR_BAD_ARG, "latent_append: unknown cache dtype %d", cache_dtype);
  NB_CHECK_LAUNCH("latent_append");
  return 0;
}

// x: [n_rows][x_stride], head h's inputs at columns x_col + h*n_in ..; W: [n_heads][n_out][n_in];
// y: [n_rows][y_stride], head h's outputs at columns h*n_out ..; gate (optional): fp32
// [n_rows][gate_stride], head h's gate logit at column gate_col + h.  Rows with a negative
// slot give zeros.
NB_EXPORT int nb_head_linear(const void* x, int x_dtype, int x_stride, int x_col, const void* W,
                             int w_dtype, void* y, int y_dtype, int y_stride, const float* gate,
                             int gate_stride, int gate_col, const int* row_slot, int n_rows,
                             int n_heads, int n_in, int n_out, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(n_heads > 0 && n_heads <= 65535 && n_in > 0 && n_out > 0, NB_ERR_BAD_ARG,
             "head_linear: bad sizes heads=%d in=%d out=%d", n_heads, n_in, n_out);
  const size_t smem = (size_t)HL_ROWS * n_in * sizeof(float);
  NB_REQUIRE(smem <= 200 * 1024, NB_ERR_UNSUPPORTED, "head_linear: %d inputs per head are too many",
             n_in);
  const dim3 grid((n_rows + HL_ROWS - 1) / HL_ROWS, n_heads);
#define NB_HL(TX, TW, TY)                                                                        \
  do {                                                                                           \
    if (smem > 48 * 1024)                                                                        \
      NB_CUDA(cudaFuncSetAttribute(head_linear_kernel<TX, TW, TY>,                               \
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));     \
    NB_CUDA(nb_launch(head_linear_kernel<TX, TW, TY>, grid, dim3(THREADS), smem, stream,         \
                      (const TX*)x, x_stride, x_col, (const TW*)W, (TY*)y, y_stride, gate,       \
                      gate_stride, gate_col, row_slot, n_rows, n_in, n_out));                    \
  } while (0)
  const int key = x_dtype * 4 + w_dtype * 2 + y_dtype;
  switch (key) {
    case 0: NB_HL(float, float, float); break;
    case 1: NB_HL(float, float, bf16); break;
    case 2: NB_HL(float, bf16, float); break;
    case 3: NB_HL(float, bf16, bf16); break;
    case 4: NB_HL(bf16, float, float); break;
    case 5: NB_HL(bf16, float, bf16); break;
    case 6: NB_HL(bf16, bf16, float); break;
    case 7: NB_HL(bf16, bf16, bf16); break;
    default: NB_REQUIRE(false, NB_ERR_BAD_ARG, "head_linear: unknown dtypes %d/%d/%d", x_dtype, w_dtype, y_dtype);
  }
#undef NB_HL
  NB_CHECK_LAUNCH("head_linear");
  return 0;
}

// q: [n_rows][q_stride], head h's query (already mapped into the latent's space) at columns
// q_col + h*rank ..; cache: one plane [n_pages][page][rank]; out: [n_rows][out_stride], head
// h at columns h*rank; sink: fp32 [n_heads] or null.
NB_EXPORT int nb_attention_latent(const void* q, int q_dtype, int q_stride, int q_col,
                                  const int* row_slot, const int* row_pos, const void* cache,
                                  int cache_dtype, const int* block_table, int max_pages, int page,
                                  int n_heads, int rank, const float* sink, void* out,
                                  int out_dtype, int out_stride, float scale, int window,
                                  int n_rows, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(rank >= 1 && rank <= MAX_ACC * THREADS, NB_ERR_UNSUPPORTED,
             "attention_latent: latent size %d is outside 1..%d", rank, MAX_ACC * THREADS);
  NB_REQUIRE(n_heads >= 1 && n_heads <= 65535 && page > 0, NB_ERR_BAD_ARG,
             "attention_latent: bad sizes heads=%d page=%d", n_heads, page);
  const size_t smem = (size_t)(rank + CHUNK) * sizeof(float);
  const dim3 grid(n_rows, n_heads);
#define NB_AL(TQ, TC, TO)                                                                        \
  NB_CUDA(nb_launch(attention_latent_kernel<TQ, TC, TO>, grid, dim3(THREADS), smem, stream,      \
                    (const TQ*)q, q_stride, q_col, row_slot, row_pos, (const TC*)cache,          \
                    block_table, max_pages, page, rank, sink, (TO*)out, out_stride, scale, window))
  const int key = q_dtype * 4 + cache_dtype * 2 + out_dtype;
  switch (key) {
    case 0: NB_AL(float, float, float); break;
    case 1: NB_AL(float, float, bf16); break;
    case 2: NB_AL(float, bf16, float); break;
    case 3: NB_AL(float, bf16, bf16); break;
    case 4: NB_AL(bf16, float, float); break;
    case 5: NB_AL(bf16, float, bf16); break;
    case 6: NB_AL(bf16, bf16, float); break;
    case 7: NB_AL(bf16, bf16, bf16); break;
    default: NB_REQUIRE(false, NB_ERR_BAD_ARG, "attention_latent: unknown dtypes %d/%d/%d", q_dtype, cache_dtype, out_dtype);
  }
#undef NB_AL
  NB_CHECK_LAUNCH("attention_latent");
  return 0;
}
