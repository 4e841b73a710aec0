// The matrix-memory recurrence of xLSTM (mLSTM) with a state slot per request.
//
// Per head, with q (scaled), k of D values, v of V values, a log input gate gi and a log forget gate gf:
//   m_t = max(gf + m_(t-1), gi)
//   S_t = exp(gf + m_(t-1) - m_t) S_(t-1) + exp(gi - m_t) k v^T        (D x V)
//   n_t = exp(gf + m_(t-1) - m_t) n_(t-1) + exp(gi - m_t) k            (D)
//   o_t = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6)                  (V)
// S, n and m start at zero (m at 0, not at minus infinity).  The gates are capped:
//   gi = cap tanh((x_i + b_i) / cap),   gf = logsigmoid(cap tanh((x_f + b_f) / cap)).
// The scan kernel walks a request's tokens of this step in order from the state its slot holds (from zero when the
// portion starts at position 0) and leaves the new state there; everything is float32, and a token's result does
// not depend on where the sequence was cut.  One block = one request x one head x MLSTM_VB columns of S; the
// blocks of a head each keep n and m (the first one stores them).  A second kernel divides each head's o by its
// root mean square and applies the weight and the output gate.
#include "common.cuh"

constexpr int MLSTM_VB = 32, MLSTM_DY = 8, MLSTM_THREADS = MLSTM_VB * MLSTM_DY;

__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

__global__ void __launch_bounds__(MLSTM_THREADS)
mlstm_scan_kernel(const float* __restrict__ proj, int64_t ld, int off_q, int off_k, int off_v, int off_i, int off_f,
                  const float* __restrict__ bias_i, const float* __restrict__ bias_f, float cap,
                  float* __restrict__ S_state, float* __restrict__ n_state, float* __restrict__ m_state,
                  const int* __restrict__ cu_seqlens, const int* __restrict__ context_lens,
                  const int* __restrict__ state_slots, float* __restrict__ o, int H, int D, int V, float q_scale) {
  extern __shared__ float smem[];
  __shared__ float red[32];
  float* S = smem;                              // [D][MLSTM_VB + 1]
  float* q_s = S + D * (MLSTM_VB + 1);          // [D]
  float* k_s = q_s + D;                         // [D]
  float* n_s = k_s + D;                         // [D]
  float* parts = n_s + D;                       // [MLSTM_DY][MLSTM_VB]
  const int b = blockIdx.x, hd = blockIdx.y, v0 = blockIdx.z * MLSTM_VB;
  const int tid = threadIdx.x, vc = tid % MLSTM_VB, dy = tid / MLSTM_VB;
  const bool v_ok = v0 + vc < V;
  const float bi = bias_i[hd], bf_ = bias_f[hd];
  pdl_wait();
  pdl_launch_dependents();
  const int slot = state_slots[b];
  const int tok0 = cu_seqlens[b], n_tok = cu_seqlens[b + 1] - tok0;
  if (slot < 0 || n_tok <= 0) return;
  const bool fresh = context_lens[b] - n_tok == 0;
  float* Sg = S_state + ((int64_t)slot * H + hd) * D * V;
  float* ng = n_state + ((int64_t)slot * H + hd) * D;
  for (int d = dy; d < D; d += MLSTM_DY) S[d * (MLSTM_VB + 1) + vc] = (fresh || !v_ok) ? 0.f : Sg[(int64_t)d * V + v0 + vc];
  for (int d = tid; d < D; d += MLSTM_THREADS) n_s[d] = fresh ? 0.f : ng[d];
  float m = fresh ? 0.f : m_state[(int64_t)slot * H + hd];
  for (int i = 0; i < n_tok; ++i) {
    const float* row = proj + (int64_t)(tok0 + i) * ld;
    __syncthreads();                            // the token before is done with q_s, k_s, parts
    for (int d = tid; d < D; d += MLSTM_THREADS) {
      q_s[d] = row[off_q + hd * D + d] * q_scale;
      k_s[d] = row[off_k + hd * D + d];
    }
    const float gi = cap * tanhf((row[off_i + hd] + bi) / cap);
    const float gf = log_sigmoid(cap * tanhf((row[off_f + hd] + bf_) / cap));
    const float m_new = fmaxf(gf + m, gi);
    const float fa = expf(gf + m - m_new), fb = expf(gi - m_new);
    const float vv = v_ok ? row[off_v + hd * V + v0 + vc] : 0.f;
    __syncthreads();
    float nq = 0.f;
    for (int d = tid; d < D; d += MLSTM_THREADS) {
      const float nn = fmaf(fa, n_s[d], fb * k_s[d]);
      n_s[d] = nn;
      nq = fmaf(nn, q_s[d], nq);
    }
    nq = block_sum(nq, red);
    float part = 0.f;
    for (int d = dy; d < D; d += MLSTM_DY) {
      const float s = fmaf(fa, S[d * (MLSTM_VB + 1) + vc], fb * k_s[d] * vv);
      S[d * (MLSTM_VB + 1) + vc] = s;
      part = fmaf(s, q_s[d], part);
    }
    parts[dy * MLSTM_VB + vc] = part;
    __syncthreads();
    if (dy == 0 && v_ok) {
      float tot = 0.f;
#pragma unroll
      for (int y = 0; y < MLSTM_DY; ++y) tot += parts[y * MLSTM_VB + vc];
      const float den = fmaxf(fabsf(nq), expf(-m_new)) + 1e-6f;
      o[(int64_t)(tok0 + i) * H * V + hd * V + v0 + vc] = tot / den;
    }
    m = m_new;
  }
  __syncthreads();
  if (v_ok)
    for (int d = dy; d < D; d += MLSTM_DY) Sg[(int64_t)d * V + v0 + vc] = S[d * (MLSTM_VB + 1) + vc];
  if (blockIdx.z == 0) {
    for (int d = tid; d < D; d += MLSTM_THREADS) ng[d] = n_s[d];
    if (tid == 0) m_state[(int64_t)slot * H + hd] = m;
  }
}

// out[t, h*V + v] = o / sqrt(mean_v(o^2) + eps) * w[h*V + v] * sigmoid(g[t, h*V + v]); one warp a head.
template <typename TO>
__global__ void __launch_bounds__(128)
mlstm_out_kernel(const float* __restrict__ o, const float* __restrict__ proj, int64_t ld, int off_g,
                 const float* __restrict__ w, float eps, TO* __restrict__ out, int H, int V) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int hd = warp; hd < H; hd += nw) {
    const float* oo = o + ((int64_t)t * H + hd) * V;
    float ss = 0.f;
    for (int v = lane; v < V; v += 32) ss = fmaf(oo[v], oo[v], ss);
    const float r = 1.0f / sqrtf(warp_sum(ss) / (float)V + eps);
    for (int v = lane; v < V; v += 32) {
      const float g = proj[(int64_t)t * ld + off_g + hd * V + v];
      out[((int64_t)t * H + hd) * V + v] = from_f<TO>(oo[v] * r * w[hd * V + v] * (1.0f / (1.0f + expf(-g))));
    }
  }
}

// proj: [T, ld] float32 rows holding q, k (H*D each), v, g (H*V each), i, f (H each) at the given column offsets.
// S_state [slots, H, D, V], n_state [slots, H, D], m_state [slots, H] float32.  o: [T, H*V] float32 work buffer.
ME_API int me_mlstm_scan(const float* proj, int64_t ld, int off_q, int off_k, int off_v, int off_i, int off_f,
                         const float* bias_i, const float* bias_f, float cap, float* S_state, float* n_state, float* m_state,
                         const int* cu_seqlens, const int* context_lens, const int* state_slots, float* o, int B, int H, int D,
                         int V, float q_scale, cudaStream_t stream) {
  if (B == 0) return 0;
  ME_REQUIRE(B > 0 && H > 0 && D > 0 && V > 0 && cap > 0.f, "me_mlstm_scan: bad sizes B=%d H=%d D=%d V=%d cap=%g", B, H, D, V, cap);
  ME_REQUIRE(H <= 65535, "me_mlstm_scan: too many heads");
  const size_t smem = sizeof(float) * ((size_t)D * (MLSTM_VB + 1) + 3 * (size_t)D + MLSTM_DY * MLSTM_VB);
  ME_REQUIRE(smem <= 200 * 1024, "me_mlstm_scan: head size %d is too large", D);
  if (smem > 48 * 1024) {
    static bool attr_set = false;
    if (!attr_set) {
      cudaError_t e = cudaFuncSetAttribute(mlstm_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      ME_REQUIRE(e == cudaSuccess, "me_mlstm_scan: cannot raise shared memory: %s", cudaGetErrorString(e));
      attr_set = true;
    }
  }
  me_launch(mlstm_scan_kernel, dim3(B, H, (V + MLSTM_VB - 1) / MLSTM_VB), dim3(MLSTM_THREADS), smem, stream, proj, ld, off_q,
            off_k, off_v, off_i, off_f, bias_i, bias_f, cap, S_state, n_state, m_state, cu_seqlens, context_lens, state_slots, o,
            H, D, V, q_scale);
  ME_LAUNCH_CHECK("me_mlstm_scan");
  return 0;
}

ME_API int me_mlstm_out(const float* o, const float* proj, int64_t ld, int off_g, const float* w, float eps, void* out,
                        int out_dtype, int T, int H, int V, cudaStream_t stream) {
  if (T == 0) return 0;
  ME_REQUIRE(T > 0 && H > 0 && V > 0, "me_mlstm_out: bad sizes T=%d H=%d V=%d", T, H, V);
  ME_DISPATCH_DTYPE(out_dtype, TO, me_launch(mlstm_out_kernel<TO>, dim3(T), dim3(128), 0, stream, o, proj, ld, off_g, w, eps,
                                             (TO*)out, H, V));
  ME_LAUNCH_CHECK("me_mlstm_out");
  return 0;
}
