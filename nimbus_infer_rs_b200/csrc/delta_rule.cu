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
// A CTA takes one (sequence, head).  Column j lives in the registers of LPC = 4 neighbouring
// lanes, a quarter of the key channels each; the two dot products finish with two shuffles.
// The channels are dealt to the four lanes in groups of four (lane q has channels 16 g + 4 q ..
// 16 g + 4 q + 3 for g = 0, 1, ...), so that the four lanes of a column read 64 consecutive
// bytes of a shared-memory vector with one 16-byte load each: no bank conflicts, and the other
// seven columns of the warp get the same bytes by broadcast.
// Tokens are taken CHUNK at a time: all threads prepare the chunk's vectors (w, a*u, u, k, r, v)
// in shared memory, then every thread walks the chunk's tokens in order without a barrier, then
// all threads norm, gate and store the chunk's outputs.  The state is read from the sequence's
// state row before the first token of the step and written back after the last, so a sequence
// may be cut into steps anywhere: the arithmetic per token does not depend on the cut, nor on
// what else is in the batch.
//
// A decode step (one token per sequence) is the same kernel with a chunk of one token: it reads
// and writes the state once, which is all the memory traffic there is.
#include "common.cuh"

namespace {

constexpr int LPC = 4;       // lanes per column of the state
constexpr int CHUNK = 16;    // tokens prepared at a time

template <int DP, typename TOut>
__global__ void __launch_bounds__(LPC * DP)
delta_rule_kernel(const float* fused, int stride, int col_r, int col_k, int col_v, int col_g,
                  int col_a, const float* decay_logits, const float* __restrict__ a_bias,
                  const float* __restrict__ norm_w, float eps, float rate, float key_eps,
                  const int* cu_rows, const int* seq_slot, float* state, TOut* out, int n_heads,
                  int d, int n_seqs, int n_rows) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  constexpr int KPL = DP / LPC;                 // key channels per lane
  constexpr int THREADS = LPC * DP;
  constexpr int NW = THREADS / 32;
  extern __shared__ __align__(16) float sm[];
  float* w_s = sm;                              // [CHUNK][DP] each
  float* au_s = w_s + CHUNK * DP;
  float* u_s = au_s + CHUNK * DP;
  float* k_s = u_s + CHUNK * DP;
  float* r_s = k_s + CHUNK * DP;
  float* v_s = r_s + CHUNK * DP;
  float* o_s = v_s + CHUNK * DP;

  const int seq = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int hd = n_heads * d;

  if (seq == 0) {   // padding rows after the last sequence give zeros
    for (int r = cu_rows[n_seqs]; r < n_rows; ++r)
      for (int i = tid; i < d; i += THREADS) out[(size_t)r * hd + h * d + i] = nb_from_f32<TOut>(0.0f);
  }
  const int row0 = cu_rows[seq], row1 = cu_rows[seq + 1];
  const int slot = seq_slot[seq];
  if (slot < 0 || row1 <= row0) return;

  const int col = tid / LPC, q = tid % LPC;     // this thread's column and quarter of the keys
  // the key channel of this thread's i-th state value
  auto channel = [q](int i) { return (((i >> 2) * LPC + q) << 2) + (i & 3); };
  float* st = state + ((size_t)slot * n_heads + h) * d * d;
  float S[KPL];
#pragma unroll
  for (int i = 0; i < KPL; ++i) {
    const int k = channel(i);
    S[i] = (k < d && col < d) ? st[(size_t)k * d + col] : 0.0f;
  }

  for (int c0 = row0; c0 < row1; c0 += CHUNK) {
    const int nc = min(CHUNK, row1 - c0);
    // ---- prepare: a warp per token, lanes over the key channels
    for (int c = warp; c < nc; c += NW) {
      const float* row = fused + (size_t)(c0 + c) * stride;
      const float* dl = decay_logits + (size_t)(c0 + c) * hd + h * d;
      float ss = 0.0f;
      for (int k = lane; k < d; k += 32) {
        const float kx = row[col_k + h * d + k];
        ss = fmaf(kx, kx, ss);
      }
      ss = nb_warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss + key_eps);
      for (int k = lane; k < DP; k += 32) {
        float wv = 0.0f, au = 0.0f, u = 0.0f, kx = 0.0f, rx = 0.0f, vx = 0.0f;
        if (k < d) {
          kx = row[col_k + h * d + k];
          rx = row[col_r + h * d + k];
          vx = row[col_v + h * d + k];
          u = kx * inv;
          const float a = nb_sigmoid(row[col_a + h * d + k] + a_bias[h * d + k]);
          au = a * u;
          wv = expf(-rate * nb_sigmoid(dl[k]));
        }
        w_s[c * DP + k] = wv;
        au_s[c * DP + k] = au;
        u_s[c * DP + k] = u;
        k_s[c * DP + k] = kx;
        r_s[c * DP + k] = rx;
        v_s[c * DP + k] = vx;
      }
    }
    __syncthreads();
    // ---- the recurrence: every thread walks the chunk's tokens in order
    for (int c = 0; c < nc; ++c) {
      const float4* w4 = reinterpret_cast<const float4*>(w_s + c * DP) + q;
      const float4* au4 = reinterpret_cast<const float4*>(au_s + c * DP) + q;
      const float4* u4 = reinterpret_cast<const float4*>(u_s + c * DP) + q;
      const float4* k4 = reinterpret_cast<const float4*>(k_s + c * DP) + q;
      const float4* r4 = reinterpret_cast<const float4*>(r_s + c * DP) + q;
      const float vj = v_s[c * DP + col];
      float rem = 0.0f;
#pragma unroll
      for (int g = 0; g < KPL / 4; ++g) {
        const float4 uu = u4[g * LPC];
        rem = fmaf(uu.x, S[4 * g], rem);
        rem = fmaf(uu.y, S[4 * g + 1], rem);
        rem = fmaf(uu.z, S[4 * g + 2], rem);
        rem = fmaf(uu.w, S[4 * g + 3], rem);
      }
      rem += __shfl_xor_sync(0xffffffffu, rem, 1);
      rem += __shfl_xor_sync(0xffffffffu, rem, 2);
      float o = 0.0f;
#pragma unroll
      for (int g = 0; g < KPL / 4; ++g) {
        const float4 ww = w4[g * LPC], aa = au4[g * LPC], kk = k4[g * LPC], rr = r4[g * LPC];
        S[4 * g] = fmaf(kk.x, vj, fmaf(ww.x, S[4 * g], -aa.x * rem));
        S[4 * g + 1] = fmaf(kk.y, vj, fmaf(ww.y, S[4 * g + 1], -aa.y * rem));
        S[4 * g + 2] = fmaf(kk.z, vj, fmaf(ww.z, S[4 * g + 2], -aa.z * rem));
        S[4 * g + 3] = fmaf(kk.w, vj, fmaf(ww.w, S[4 * g + 3], -aa.w * rem));
        o = fmaf(S[4 * g], rr.x, o);
        o = fmaf(S[4 * g + 1], rr.y, o);
        o = fmaf(S[4 * g + 2], rr.z, o);
        o = fmaf(S[4 * g + 3], rr.w, o);
      }
      o += __shfl_xor_sync(0xffffffffu, o, 1);
      o += __shfl_xor_sync(0xffffffffu, o, 2);
      if (q == 0) o_s[c * DP + col] = o;
    }
    __syncthreads();
    // ---- norm over the head, weight, gate, store: a warp per token
    for (int c = warp; c < nc; c += NW) {
      float ss = 0.0f;
      for (int j = lane; j < d; j += 32) {
        const float o = o_s[c * DP + j];
        ss = fmaf(o, o, ss);
      }
      ss = nb_warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss / (float)d + eps);
      const float* row = fused + (size_t)(c0 + c) * stride;
      for (int j = lane; j < d; j += 32) {
        const float g = nb_sigmoid(row[col_g + h * d + j]);
        out[(size_t)(c0 + c) * hd + h * d + j] =
            nb_from_f32<TOut>(o_s[c * DP + j] * inv * norm_w[h * d + j] * g);
      }
    }
    // the next chunk's preparation writes other arrays than the ones read above, and its
    // barrier stands between these reads of o_s and the next writes to it
  }
#pragma unroll
  for (int i = 0; i < KPL; ++i) {
    const int k = channel(i);
    if (k < d && col < d) st[(size_t)k * d + col] = S[i];
  }
}

template <int DP, typename TOut>
int launch(cudaStream_t stream, const float* fused, int stride, int col_r, int col_k, int col_v,
           int col_g, int col_a, const float* decay_logits, const float* a_bias,
           const float* norm_w, float eps, float rate, float key_eps, const int* cu_rows,
           const int* seq_slot, float* state, void* out, int n_heads, int d, int n_seqs,
           int n_rows) {
  const size_t smem = (size_t)7 * CHUNK * DP * sizeof(float);
  auto kern = delta_rule_kernel<DP, TOut>;
  if (smem > 48 * 1024)
    NB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  NB_CUDA(nb_launch(kern, dim3(n_seqs, n_heads), dim3(LPC * DP), smem, stream, fused, stride, col_r,
                    col_k, col_v, col_g, col_a, decay_logits, a_bias, norm_w, eps, rate, key_eps,
                    cu_rows, seq_slot, state, (TOut*)out, n_heads, d, n_seqs, n_rows));
  return 0;
}

}  // namespace

NB_EXPORT int nb_delta_rule_supported(int d) { return d >= 1 && d <= 256 ? 1 : 0; }

// fused: fp32 [n_rows][stride] with head h's r, k, v, gate logits and a logits at columns
// col_x + h*d ..; decay_logits: fp32 [n_rows][n_heads*d]; a_bias, norm_w: fp32 [n_heads*d];
// state: fp32 [n_slots][n_heads][d][d] (key channel, value channel); out: [n_rows][n_heads*d].
// cu_rows [n_seqs+1], seq_slot [n_seqs]: the packed batch.
NB_EXPORT int nb_delta_rule(const float* fused, int stride, int col_r, int col_k, int col_v,
                            int col_g, int col_a, const float* decay_logits, const float* a_bias,
                            const float* norm_w, float eps, float rate, float key_eps,
                            const int* cu_rows, const int* seq_slot, float* state, void* out,
                            int out_dtype, int n_heads, int d, int n_seqs, int n_rows,
                            cudaStream_t stream) {
  if (n_rows == 0 || n_seqs == 0) return 0;
  NB_REQUIRE(n_heads >= 1 && n_heads <= 65535 && n_seqs > 0 && n_rows > 0, NB_ERR_BAD_ARG,
             "delta_rule: bad sizes heads=%d seqs=%d rows=%d", n_heads, n_seqs, n_rows);
  NB_REQUIRE(d >= 1 && d <= 256, NB_ERR_UNSUPPORTED,
             "delta_rule: heads of %d channels are outside 1..256", d);
  NB_REQUIRE(out_dtype == NB_F32 || out_dtype == NB_BF16, NB_ERR_BAD_ARG,
             "delta_rule: unknown output dtype %d", out_dtype);
  int rc;
#define NB_DR(DP)                                                                                 \
  rc = out_dtype == NB_F32                                                                        \
           ? launch<DP, float>(stream, fused, stride, col_r, col_k, col_v, col_g, col_a,          \
                               decay_logits, a_bias, norm_w, eps, rate, key_eps, cu_rows,         \
                               seq_slot, state, out, n_heads, d, n_seqs, n_rows)                  \
           : launch<DP, __nv_bfloat16>(stream, fused, stride, col_r, col_k, col_v, col_g, col_a,  \
                                       decay_logits, a_bias, norm_w, eps, rate, key_eps, cu_rows, \
                                       seq_slot, state, out, n_heads, d, n_seqs, n_rows)
  if (d <= 32) NB_DR(32);
  else if (d <= 64) NB_DR(64);
  else if (d <= 128) NB_DR(128);
  else NB_DR(256);
#undef NB_DR
  if (rc != 0) return rc;
  NB_CHECK_LAUNCH("delta_rule");
  return 0;
}
