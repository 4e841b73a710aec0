// What lies between the packed q|k|v projection and the attention kernel of a mixer whose projections pass through a
// short causal convolution: bias, convolution over time with the last inputs of every request as state, rotation of
// neighbouring pairs, and the write of the new keys and values into the paged cache, in one pass.
//
// u_t = proj_t + bias (zeros before a request's first token), y_t = sum_j w[:, j] * u_(t - taps + 1 + j), j < taps.
// Channels are laid out q (nh x D) | k (nkv x D) | v (nkv x Dv); a mixer that takes its keys and values from another
// layer has only q.  Of every q and k head the first ``rot`` elements are rotated, (2i, 2i+1) by the angle
// position * inv_freq[i]: the angle is formed in double precision and brought into [-pi, pi] there, so that the float32
// sine and cosine are as exact at position 100,000 as at position 1.  The cache is the
// engine's usual one, [page][keys | values][kv head][page offset][HD] with HD >= max(D, Dv); a key fills the first D
// elements of its row, a value the first Dv of its own.
// The state [slots][taps-1][channels] (float32) holds u at the last taps-1 positions; it is read for positions before the
// portion's first token and renewed by a second kernel.  No slot is read for positions below 0.
#include "common.cuh"

struct ConvSrc {
  const float* proj; int64_t stride;      // [T, >= C] float32
  const float* bias;                      // [C] or null
  const float* state;                     // [slots, taps-1, C] or null
  int C, taps;
};

// u of channel c at local index src (may be negative: from the state) of a portion that starts at position ``start``.
__device__ __forceinline__ float conv_input(const ConvSrc& s, int tok0, int src, int start, int slot, int c) {
  if (start + src < 0) return 0.f;
  if (src >= 0) return s.proj[(int64_t)(tok0 + src) * s.stride + c] + (s.bias ? s.bias[c] : 0.f);
  if (slot < 0) return 0.f;
  return s.state[((int64_t)slot * (s.taps - 1) + (src + s.taps - 1)) * s.C + c];
}

__device__ __forceinline__ float conv_output(const ConvSrc& s, const float* __restrict__ wt, int tok0, int i, int start, int slot,
                                             int c) {
  if (!wt) return conv_input(s, tok0, i, start, slot, c);
  float acc = 0.f;
  for (int j = 0; j < s.taps; ++j) acc = fmaf(wt[(int64_t)c * s.taps + j], conv_input(s, tok0, i - (s.taps - 1) + j, start, slot, c), acc);
  return acc;
}

// Where channel c of token t goes: a query element, or (through the slot mapping) an element of a cached key or value.
template <typename TO>
__device__ __forceinline__ void conv_store(float y, int c, int t, int where, TO* __restrict__ q_out, TO* __restrict__ pool, int Cq,
                                           int Ck, int nkv, int D, int Dv, int HD, int page_size) {
  if (c < Cq) {
    q_out[(int64_t)t * Cq + c] = from_f<TO>(y);
    return;
  }
  if (where < 0) return;
  const int page = where / page_size, off = where - page * page_size;
  int g, e, which;
  if (c < Cq + Ck) { which = 0; g = (c - Cq) / D; e = (c - Cq) - g * D; }
  else { which = 1; g = (c - Cq - Ck) / Dv; e = (c - Cq - Ck) - g * Dv; }
  pool[((((int64_t)page * 2 + which) * nkv + g) * page_size + off) * HD + e] = from_f<TO>(y);
}

// A thread owns two neighbouring channels (2i, 2i+1): with an even head size they are a rotated pair or no part of one.
template <typename TO>
__global__ void __launch_bounds__(256)
conv_rope_kv_kernel(ConvSrc s, const float* __restrict__ wt, const double* __restrict__ inv_freq, int rot,
                    const int* __restrict__ positions, const int* __restrict__ token_req, const int* __restrict__ cu_seqlens,
                    const int* __restrict__ context_lens, const int* __restrict__ state_slots,
                    const int* __restrict__ slot_mapping, TO* __restrict__ q_out, TO* __restrict__ pool, int nh, int nkv, int D,
                    int Dv, int HD, int page_size, float* __restrict__ state_out, int vec2) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int c = 2 * (blockIdx.y * blockDim.x + threadIdx.x);
  if (c >= s.C) return;
  const bool two = c + 1 < s.C;
  const int b = token_req[t];
  const int tok0 = cu_seqlens[b], q_len = cu_seqlens[b + 1] - tok0;
  const int start = context_lens[b] - q_len;
  const int i = t - tok0;
  const int slot = state_slots[b];
  const int Cq = nh * D, Ck = nkv * D;
  float y0, y1 = 0.f;
  if (two && i >= s.taps - 1) {
    // The usual case, all taps inside this step's rows: no state, no start of the sequence, one address a tap.
    const float* row = s.proj + (int64_t)t * s.stride + c;
    const float b0 = s.bias ? s.bias[c] : 0.f, b1 = s.bias ? s.bias[c + 1] : 0.f;
    if (!wt) {
      y0 = row[0] + b0;
      y1 = row[1] + b1;
    } else {
      const float* w0 = wt + (int64_t)c * s.taps;
      const float* w1 = w0 + s.taps;
      y0 = 0.f;
      for (int j = 0; j < s.taps; ++j) {
        const float* u = row - (int64_t)(s.taps - 1 - j) * s.stride;
        float u0, u1;
        if (vec2) {
          const float2 v = *reinterpret_cast<const float2*>(u);
          u0 = v.x;
          u1 = v.y;
        } else {
          u0 = u[0];
          u1 = u[1];
        }
        y0 = fmaf(w0[j], u0 + b0, y0);
        y1 = fmaf(w1[j], u1 + b1, y1);
      }
    }
  } else {
    y0 = conv_output(s, wt, tok0, i, start, slot, c);
    if (two) y1 = conv_output(s, wt, tok0, i, start, slot, c + 1);
  }
  if (rot > 0 && c < Cq + Ck) {
    const int d = (c < Cq ? c : c - Cq) % D;        // even, since D is even when anything is rotated
    if (d < rot) {
      // the angle in double precision, brought into [-pi, pi] there, then the float32 sine and cosine of that
      double ang = (double)positions[t] * inv_freq[d >> 1];
      ang -= 6.283185307179586476925 * rint(ang * 0.15915494309189533577);
      float sn, cs;
      sincosf((float)ang, &sn, &cs);
      const float u = y0, v = y1;
      y0 = fmaf(u, cs, -v * sn);
      y1 = fmaf(v, cs, u * sn);
    }
  }
  const int where = slot_mapping ? slot_mapping[t] : -1;
  conv_store<TO>(y0, c, t, where, q_out, pool, Cq, Ck, nkv, D, Dv, HD, page_size);
  if (two) conv_store<TO>(y1, c + 1, t, where, q_out, pool, Cq, Ck, nkv, D, Dv, HD, page_size);
  // A step in which every request brings one token: no other thread reads these channels of this slot, so the state moves
  // on here (rows up by one, the newest u last) and the second kernel is not launched.
  if (state_out && slot >= 0 && q_len == 1) {
    for (int cc = c; cc < c + (two ? 2 : 1); ++cc) {
      float* st = state_out + (int64_t)slot * (s.taps - 1) * s.C + cc;
      for (int k = 0; k < s.taps - 1; ++k) st[(int64_t)k * s.C] = conv_input(s, tok0, k - (s.taps - 2), start, slot, cc);
    }
  }
}

__global__ void __launch_bounds__(256)
conv_state_kernel(ConvSrc s, float* __restrict__ state, const int* __restrict__ cu_seqlens, const int* __restrict__ context_lens,
                  const int* __restrict__ state_slots) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= s.C) return;
  const int slot = state_slots[b];
  if (slot < 0) return;
  const int tok0 = cu_seqlens[b], n = cu_seqlens[b + 1] - tok0;
  if (n <= 0) return;
  const int start = context_lens[b] - n;
  float* st = state + (int64_t)slot * (s.taps - 1) * s.C + c;
  // Row k takes u at local index n - (taps-1) + k.  Old rows are read at k + n > k and rows are written in ascending
  // order, so a thread never reads a row that it has replaced.
  for (int k = 0; k < s.taps - 1; ++k) st[(int64_t)k * s.C] = conv_input(s, tok0, n - (s.taps - 1) + k, start, slot, c);
}

// proj: [T, >= C] float32 with C = nh*D + (own_kv ? nkv*(D+Dv) : 0) leading channels q|k|v.  bias: [C] or null.  wt: [C, taps]
// or null (no convolution; taps is then 1).  state: [slots, taps-1, C] float32 (unused for taps == 1).  inv_freq: [rot/2]
// float64.  single_tokens != 0: every request of the step brings one token (T == B); the state then moves on in the first
// kernel.  q_out: [T, nh*D]; pool: [pages][2][nkv][page_size][HD] of out_dtype (unused without own_kv).
ME_API int me_conv_rope_kv(const float* proj, int64_t proj_stride, const float* bias, const float* wt, float* state, int taps,
                           const double* inv_freq, int rot, const int* positions, const int* token_req, const int* cu_seqlens,
                           const int* context_lens, const int* state_slots, const int* slot_mapping, void* q_out, void* pool,
                           int out_dtype, int T, int B, int nh, int nkv, int D, int Dv, int HD, int own_kv, int page_size,
                           int single_tokens, cudaStream_t stream) {
  if (T == 0) return 0;
  ME_REQUIRE(T > 0 && B > 0 && nh > 0 && D > 0 && taps >= 1, "me_conv_rope_kv: bad sizes");
  ME_REQUIRE(rot % 2 == 0 && rot >= 0 && rot <= D && (rot == 0 || D % 2 == 0), "me_conv_rope_kv: %d of %d elements rotated", rot, D);
  ME_REQUIRE(taps == 1 || (state != nullptr && wt != nullptr), "me_conv_rope_kv: %d taps need weights and a state", taps);
  ConvSrc s{proj, proj_stride, bias, state, nh * D + (own_kv ? nkv * (D + Dv) : 0), taps};
  const int threads = s.C >= 256 ? 256 : 64;
  dim3 grid(T, ((s.C + 1) / 2 + threads - 1) / threads);
  ME_DISPATCH_DTYPE(out_dtype, TO,
                    me_launch(conv_rope_kv_kernel<TO>, grid, dim3(threads), 0, stream, s, wt, inv_freq, rot, positions, token_req,
                              cu_seqlens, context_lens, state_slots, own_kv ? slot_mapping : (const int*)nullptr, (TO*)q_out,
                              (TO*)pool, nh, own_kv ? nkv : 0, D, Dv, HD, page_size,
                              (taps > 1 && single_tokens) ? state : (float*)nullptr,
                              (proj_stride % 2 == 0 && ((uintptr_t)proj & 7) == 0) ? 1 : 0));
  ME_LAUNCH_CHECK("me_conv_rope_kv");
  if (taps > 1 && !single_tokens) {
    me_launch(conv_state_kernel, dim3(B, (s.C + threads - 1) / threads), dim3(threads), 0, stream, s, state, cu_seqlens,
              context_lens, state_slots);
    ME_LAUNCH_CHECK("me_conv_rope_kv (state)");
  }
  return 0;
}
