// The generalized delta rule: a linear recurrence over a sequence's tokens with a matrix state
// per head (key channels x value channels, fp32).
//
//   S_t = diag(w_t) S_(t-1) - (a_t * u_t) (u_t^T S_(t-1)) + k_t v_t^T,      o_t = S_t^T r_t
//
// w = exp(-rate * sigmoid(decay logits)), a = sigmoid(a logits + a_bias), u = k / sqrt(sum k^2 +
// key_eps), all per head and key channel and all in fp32; the decayed and the removed term both
// read the old state.  Afterwards each head's o is divided by its root mean square (eps inside
// the root), multiplied by a weight and by sigmoid(gate logits), and written in the output type.
//
// The columns of S are independent of one another: column j follows
//   s_j <- w * s_j - (a*u) (u . s_j) + k v_j,     o_j = s_j . r.
// A CTA of 256 threads takes COLS = 256 / LPC columns of one (sequence, head); the CTAs of a
// head share nothing.  Column j lives in the registers of LPC neighbouring lanes, DP / LPC key
// channels each; the two dot products finish with log2(LPC) shuffles.  The channels are dealt to
// the lanes in groups of four (lane q has channels 4 LPC g + 4 q .. + 3 for g = 0, 1, ...), so
// that the lanes of a column read consecutive 16-byte pieces of a shared-memory vector: no bank
// conflicts, and the other columns of the warp get the same bytes by broadcast.
// Tokens are taken CHUNK at a time: all threads prepare the chunk's vectors (w, a*u, u, k, r and
// the CTA's part of v) in shared memory, a warp per token with one trip to memory; then every
// thread walks the chunk's tokens in order without a barrier; then the chunk's o goes out in
// fp32, each lane's part of it added up there (not with shuffles inside the chain from one
// token's state to the next).  A second kernel norms each head's o, applies weight and gate and writes the output type
// (the norm needs all of a head's columns).  The state is read from the sequence's state row
// before the first token of the step and written back after the last, so a sequence may be cut
// into steps anywhere: the arithmetic per token does not depend on the cut, nor on what else is
// in the batch.
//
// A decode step (one token per sequence) is the same kernel with a chunk of one token: it reads
// and writes the state once, which is all the memory traffic there is.
#include "common.cuh"

namespace {

constexpr int THREADS = 256;
constexpr int NW = THREADS / 32;
constexpr int CHUNK = 16;    // tokens prepared at a time

template <int DP, int LPC>
__global__ void __launch_bounds__(THREADS)
delta_rule_kernel(const float* fused, int stride, int col_r, int col_k, int col_v, int col_a,
                  const float* decay_logits, const float* __restrict__ a_bias, float rate,
                  float key_eps, const int* cu_rows, const int* seq_slot, float* state,
                  float* o_raw, int n_heads, int d) {
  nb_grid_dependency_wait();
  constexpr int KPL = DP / LPC;                 // key channels per lane
  constexpr int COLS = THREADS / LPC;           // columns of the state per CTA
  constexpr int KIT = DP / 32;                  // key channels per lane of a preparing warp
  static_assert(KPL % 4 == 0 && KPL >= 4, "a lane takes its channels four at a time");
  extern __shared__ __align__(16) float sm[];
  float* w_s = sm;                              // [CHUNK][DP] each
  float* au_s = w_s + CHUNK * DP;
  float* u_s = au_s + CHUNK * DP;
  float* k_s = u_s + CHUNK * DP;
  float* r_s = k_s + CHUNK * DP;
  float* v_s = r_s + CHUNK * DP;                // [CHUNK][COLS]
  float* o_s = v_s + CHUNK * COLS;              // [CHUNK][COLS][LPC]: every lane's part of o

  const int seq = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * COLS, tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int hd = n_heads * d;
  const int row0 = cu_rows[seq], row1 = cu_rows[seq + 1];
  const int slot = seq_slot[seq];
  if (slot < 0 || row1 <= row0) return;

  const int col = col0 + tid / LPC, q = tid % LPC;   // this thread's column and share of the keys
  // the key channel of this thread's i-th state value
  auto channel = [q](int i) { return (((i >> 2) * LPC + q) << 2) + (i & 3); };
  float* st = state + ((size_t)slot * n_heads + h) * d * d;
  float S[KPL];
#pragma unroll
  for (int i = 0; i < KPL; ++i) {
    const int k = channel(i);
    S[i] = (k < d && col < d) ? st[(size_t)k * d + col] : 0.0f;
  }

  // A warp prepares the tokens warp and warp + NW of a chunk.  Their rows are fetched into
  // registers a chunk ahead (PREFETCH), so that the trip to memory runs under the recurrence.
  constexpr int TPW = CHUNK / NW;
  constexpr bool PREFETCH = DP <= 128;
  float kx[TPW][KIT], rx[TPW][KIT], al[TPW][KIT], dx[TPW][KIT], vx[TPW][(COLS + 31) / 32];
  auto fetch = [&](int c0) {
#pragma unroll
    for (int t = 0; t < TPW; ++t) {
      const int r = c0 + warp + t * NW;
      const bool live = r < row1;
      const float* row = fused + (size_t)(live ? r : row0) * stride + h * d;
      const float* dl = decay_logits + (size_t)(live ? r : row0) * hd + h * d;
#pragma unroll
      for (int j = 0; j < KIT; ++j) {
        const int k = lane + 32 * j;
        const bool in = live && k < d;
        kx[t][j] = in ? row[col_k + k] : 0.0f;
        rx[t][j] = in ? row[col_r + k] : 0.0f;
        al[t][j] = in ? row[col_a + k] : 0.0f;
        dx[t][j] = in ? dl[k] : 0.0f;
      }
#pragma unroll
      for (int j = 0; j < (COLS + 31) / 32; ++j) {
        const int c = lane + 32 * j;
        vx[t][j] = (live && c < COLS && col0 + c < d) ? row[col_v + col0 + c] : 0.0f;
      }
    }
  };
  if (PREFETCH) fetch(row0);

  for (int c0 = row0; c0 < row1; c0 += CHUNK) {
    const int nc = min(CHUNK, row1 - c0);
    // ---- prepare: a warp per token, lanes over the key channels
    if (!PREFETCH) fetch(c0);
#pragma unroll
    for (int t = 0; t < TPW; ++t) {
      const int c = warp + t * NW;
      if (c >= nc) continue;
      float ss = 0.0f;
#pragma unroll
      for (int j = 0; j < KIT; ++j) ss = fmaf(kx[t][j], kx[t][j], ss);
      ss = nb_warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss + key_eps);
#pragma unroll
      for (int j = 0; j < KIT; ++j) {
        const int k = lane + 32 * j;
        const bool in = k < d;
        const float u = kx[t][j] * inv;
        const float a = in ? nb_sigmoid(al[t][j] + a_bias[h * d + k]) : 0.0f;
        w_s[c * DP + k] = in ? expf(-rate * nb_sigmoid(dx[t][j])) : 0.0f;
        au_s[c * DP + k] = a * u;
        u_s[c * DP + k] = u;
        k_s[c * DP + k] = kx[t][j];
        r_s[c * DP + k] = rx[t][j];
      }
#pragma unroll
      for (int j = 0; j < (COLS + 31) / 32; ++j) {
        const int cc = lane + 32 * j;
        if (cc < COLS) v_s[c * COLS + cc] = vx[t][j];
      }
    }
    __syncthreads();
    if (PREFETCH && c0 + CHUNK < row1) fetch(c0 + CHUNK);
    // ---- the recurrence: every thread walks the chunk's tokens in order
#pragma unroll 2
    for (int c = 0; c < nc; ++c) {
      const float4* w4 = reinterpret_cast<const float4*>(w_s + c * DP) + q;
      const float4* au4 = reinterpret_cast<const float4*>(au_s + c * DP) + q;
      const float4* u4 = reinterpret_cast<const float4*>(u_s + c * DP) + q;
      const float4* k4 = reinterpret_cast<const float4*>(k_s + c * DP) + q;
      const float4* r4 = reinterpret_cast<const float4*>(r_s + c * DP) + q;
      const float vj = v_s[c * COLS + tid / LPC];
      float r0 = 0.0f, r1 = 0.0f, r2 = 0.0f, r3 = 0.0f;     // four chains, added up at the end
#pragma unroll
      for (int g = 0; g < KPL / 4; ++g) {
        const float4 uu = u4[g * LPC];
        r0 = fmaf(uu.x, S[4 * g], r0);
        r1 = fmaf(uu.y, S[4 * g + 1], r1);
        r2 = fmaf(uu.z, S[4 * g + 2], r2);
        r3 = fmaf(uu.w, S[4 * g + 3], r3);
      }
      float rem = (r0 + r1) + (r2 + r3);
#pragma unroll
      for (int m = 1; m < LPC; m <<= 1) rem += __shfl_xor_sync(0xffffffffu, rem, m);
      float o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f;
#pragma unroll
      for (int g = 0; g < KPL / 4; ++g) {
        const float4 ww = w4[g * LPC], aa = au4[g * LPC], kk = k4[g * LPC], rr = r4[g * LPC];
        S[4 * g] = fmaf(kk.x, vj, fmaf(ww.x, S[4 * g], -aa.x * rem));
        S[4 * g + 1] = fmaf(kk.y, vj, fmaf(ww.y, S[4 * g + 1], -aa.y * rem));
        S[4 * g + 2] = fmaf(kk.z, vj, fmaf(ww.z, S[4 * g + 2], -aa.z * rem));
        S[4 * g + 3] = fmaf(kk.w, vj, fmaf(ww.w, S[4 * g + 3], -aa.w * rem));
        o0 = fmaf(S[4 * g], rr.x, o0);
        o1 = fmaf(S[4 * g + 1], rr.y, o1);
        o2 = fmaf(S[4 * g + 2], rr.z, o2);
        o3 = fmaf(S[4 * g + 3], rr.w, o3);
      }
      // this lane's part of o; the lanes' parts are added up when the chunk goes out, off the
      // chain from one token's state to the next
      o_s[c * THREADS + tid] = (o0 + o1) + (o2 + o3);
    }
    __syncthreads();
    // ---- the chunk's o, in rows of COLS consecutive floats
    for (int e = tid; e < nc * COLS; e += THREADS) {
      const int c = e / COLS, j = e - c * COLS;
      const float* part = o_s + c * THREADS + j * LPC;
      float o = 0.0f;
#pragma unroll
      for (int m = 0; m < LPC; ++m) o += part[m];
      if (col0 + j < d) o_raw[(size_t)(c0 + c) * hd + h * d + col0 + j] = o;
    }
    // the next chunk's preparation writes other arrays than o_s, and its barrier stands between
    // these reads of o_s and the next writes to it
  }
  nb_launch_dependents();
#pragma unroll
  for (int i = 0; i < KPL; ++i) {
    const int k = channel(i);
    if (k < d && col < d) st[(size_t)k * d + col] = S[i];
  }
}

// out[r, h, :] = o[r, h, :] / sqrt(mean(o[r, h, :]^2) + eps) * norm_w[h, :] * sigmoid(gate logits).
// A CTA per row, its warps over the heads; padding rows give zeros.
template <typename TOut>
__global__ void __launch_bounds__(128)
delta_finish_kernel(const float* o_raw, const float* fused, int stride, int col_g,
                    const float* __restrict__ norm_w, float eps, const int* row_slot, TOut* out,
                    int n_heads, int d) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int hd = n_heads * d;
  const bool live = row_slot[r] >= 0;
  for (int h = warp; h < n_heads; h += 4) {
    TOut* dst = out + (size_t)r * hd + h * d;
    if (!live) {
      for (int j = lane; j < d; j += 32) dst[j] = nb_from_f32<TOut>(0.0f);
      continue;
    }
    const float* o = o_raw + (size_t)r * hd + h * d;
    const float* g = fused + (size_t)r * stride + col_g + h * d;
    float ss = 0.0f;
    for (int j = lane; j < d; j += 32) ss = fmaf(o[j], o[j], ss);
    ss = nb_warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
    for (int j = lane; j < d; j += 32)
      dst[j] = nb_from_f32<TOut>(o[j] * inv * norm_w[h * d + j] * nb_sigmoid(g[j]));
  }
}

template <int DP, int LPC>
int launch(cudaStream_t stream, const float* fused, int stride, int col_r, int col_k, int col_v,
           int col_a, const float* decay_logits, const float* a_bias, float rate, float key_eps,
           const int* cu_rows, const int* seq_slot, float* state, float* o_raw, int n_heads, int d,
           int n_seqs, bool long_walk) {
  constexpr int COLS = THREADS / LPC;
  const size_t smem = (size_t)(5 * CHUNK * DP + CHUNK * COLS + CHUNK * THREADS) * sizeof(float);
  auto kern = delta_rule_kernel<DP, LPC>;
  if (smem > 48 * 1024)
    NB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const dim3 grid(n_seqs, n_heads, (d + COLS - 1) / COLS);
  // a prompt's walk runs long on few CTAs: it never overlaps its predecessor (nb_launch_serial)
  if (long_walk)
    NB_CUDA(nb_launch_serial(kern, grid, dim3(THREADS), smem, stream, fused, stride, col_r, col_k,
                             col_v, col_a, decay_logits, a_bias, rate, key_eps, cu_rows, seq_slot,
                             state, o_raw, n_heads, d));
  else
    NB_CUDA(nb_launch(kern, grid, dim3(THREADS), smem, stream, fused, stride, col_r, col_k, col_v,
                      col_a, decay_logits, a_bias, rate, key_eps, cu_rows, seq_slot, state, o_raw,
                      n_heads, d));
  return 0;
}

}  // namespace

NB_EXPORT int nb_delta_rule_supported(int d) { return d >= 1 && d <= 256 ? 1 : 0; }

// fused: fp32 [n_rows][stride] with head h's r, k, v, gate logits and a logits at columns
// col_x + h*d ..; decay_logits: fp32 [n_rows][n_heads*d]; a_bias, norm_w: fp32 [n_heads*d];
// state: fp32 [n_slots][n_heads][d][d] (key channel, value channel); o_raw: fp32 scratch
// [n_rows][n_heads*d]; out: [n_rows][n_heads*d].  cu_rows [n_seqs+1], seq_slot [n_seqs],
// row_slot [n_rows]: the packed batch.
NB_EXPORT int nb_delta_rule(const float* fused, int stride, int col_r, int col_k, int col_v,
                            int col_g, int col_a, const float* decay_logits, const float* a_bias,
                            const float* norm_w, float eps, float rate, float key_eps,
                            const int* cu_rows, const int* seq_slot, const int* row_slot,
                            float* state, float* o_raw, void* out, int out_dtype, int n_heads,
                            int d, int n_seqs, int n_rows, cudaStream_t stream) {
  if (n_rows == 0 || n_seqs == 0) return 0;
  NB_REQUIRE(n_heads >= 1 && n_heads <= 65535 && n_seqs > 0 && n_rows > 0, NB_ERR_BAD_ARG,
             "delta_rule: bad sizes heads=%d seqs=%d rows=%d", n_heads, n_seqs, n_rows);
  NB_REQUIRE(d >= 1 && d <= 256, NB_ERR_UNSUPPORTED,
             "delta_rule: heads of %d channels are outside 1..256", d);
  NB_REQUIRE(out_dtype == NB_F32 || out_dtype == NB_BF16, NB_ERR_BAD_ARG,
             "delta_rule: unknown output dtype %d", out_dtype);
  int rc;
#define NB_DR(DP, LPC)                                                                            \
  rc = launch<DP, LPC>(stream, fused, stride, col_r, col_k, col_v, col_a, decay_logits, a_bias,   \
                       rate, key_eps, cu_rows, seq_slot, state, o_raw, n_heads, d, n_seqs,        \
                       n_rows > 4 * n_seqs)
  // Lanes per column, as measured on prompts of 1,024 tokens: 16 (four channels a lane) up to
  // 64 channels, 8 above (two and four lanes a column, and four columns a thread with the
  // token's vectors shared among them, were slower: fewer warps in flight).  A CTA takes 16 or
  // 32 of a head's columns, so a head is spread over 2 to 8 CTAs.
  if (d <= 32) NB_DR(32, 8);
  else if (d <= 64) NB_DR(64, 16);
  else if (d <= 128) NB_DR(128, 8);
  else NB_DR(256, 8);
#undef NB_DR
  if (rc != 0) return rc;
  NB_CHECK_LAUNCH("delta_rule");
  if (out_dtype == NB_F32)
    NB_CUDA(nb_launch(delta_finish_kernel<float>, dim3(n_rows), dim3(128), 0, stream, o_raw, fused,
                      stride, col_g, norm_w, eps, row_slot, (float*)out, n_heads, d));
  else
    NB_CUDA(nb_launch(delta_finish_kernel<__nv_bfloat16>, dim3(n_rows), dim3(128), 0, stream, o_raw,
                      fused, stride, col_g, norm_w, eps, row_slot, (__nv_bfloat16*)out, n_heads, d));
  NB_CHECK_LAUNCH("delta_finish");
  return 0;
}
