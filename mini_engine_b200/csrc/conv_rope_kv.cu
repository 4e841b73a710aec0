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

// The angle position x frequency in double precision, brought into [-pi, pi] there, then the float32 cosine and sine of that.
__device__ __forceinline__ void rope_angle(int position, double freq, float* cs, float* sn) {
  double ang = (double)position * freq;
  ang -= 6.283185307179586476925 * rint(ang * 0.15915494309189533577);
  sincosf((float)ang, sn, cs);
}

// (cosine, sine) of every token's angles, once per step for all layers and heads that share the rotation.
__global__ void __launch_bounds__(256)
rope_table_kernel(const int* __restrict__ positions, const double* __restrict__ inv_freq, int half, int T, float2* __restrict__ out) {
  pdl_wait();
  pdl_launch_dependents();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= T * half) return;
  const int t = idx / half, i = idx - t * half;
  float cs, sn;
  rope_angle(positions[t], inv_freq[i], &cs, &sn);
  out[idx] = make_float2(cs, sn);
}

ME_API int me_rope_table(const int* positions, const double* inv_freq, int half, int T, float* out, cudaStream_t stream) {
  if (T * half == 0) return 0;
  me_launch(rope_table_kernel, dim3((T * half + 255) / 256), dim3(256), 0, stream, positions, inv_freq, half, T, (float2*)out);
  ME_LAUNCH_CHECK("me_rope_table");
  return 0;
}

constexpr int CR_TOKENS = 8;     // tokens a thread walks in a long step (one in a short step, which wants many blocks)

template <typename TO> __device__ __forceinline__ void store_pair(TO* dst, float y0, float y1, bool vec);
template <> __device__ __forceinline__ void store_pair<float>(float* dst, float y0, float y1, bool vec) {
  if (vec) *reinterpret_cast<float2*>(dst) = make_float2(y0, y1);
  else { dst[0] = y0; dst[1] = y1; }
}
template <> __device__ __forceinline__ void store_pair<bf16>(bf16* dst, float y0, float y1, bool vec) {
  if (vec) *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(y0, y1);
  else { dst[0] = __float2bfloat16_rn(y0); dst[1] = __float2bfloat16_rn(y1); }
}

// A thread owns two neighbouring channels (2i, 2i+1) -- with an even head size they are a rotated pair or no part of one --
// over CR_TOKENS consecutive tokens: what depends on the channel alone (bias, the taps' weights, the frequency, where the
// results go) is worked out once, and while the tokens stay inside one request's rows of this step the taps' inputs slide
// through registers, one new row a token.  TAPS: the number of taps (0: no convolution) when it is 0 to 4, else -1 (any
// number, every input fetched through conv_input).
template <typename TO, int TAPS>
__global__ void __launch_bounds__(256)
conv_rope_kv_kernel(ConvSrc s, const float* __restrict__ wt, const double* __restrict__ inv_freq, int rot,
                    const int* __restrict__ positions, const int* __restrict__ token_req, const int* __restrict__ cu_seqlens,
                    const int* __restrict__ context_lens, const int* __restrict__ state_slots,
                    const int* __restrict__ slot_mapping, TO* __restrict__ q_out, TO* __restrict__ pool, int nh, int nkv, int D,
                    int Dv, int HD, int page_size, float* __restrict__ state_out, int vec2, int T,
                    const float2* __restrict__ angles, int tokens_a_thread) {
  constexpr int NT = TAPS > 0 ? TAPS : 1;
  const int c = 2 * (blockIdx.y * blockDim.x + threadIdx.x);
  if (c >= s.C) return;
  const bool two = c + 1 < s.C;
  const int Cq = nh * D, Ck = nkv * D;
  // ---- per channel pair (weights and tables are not written by this step) ----
  const float b0 = s.bias ? s.bias[c] : 0.f, b1 = (s.bias && two) ? s.bias[c + 1] : 0.f;
  float w0[NT], w1[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    w0[j] = (TAPS > 0) ? wt[(int64_t)c * TAPS + j] : 1.f;
    w1[j] = (TAPS > 0 && two) ? wt[(int64_t)(c + 1) * TAPS + j] : 1.f;
  }
  // where the pair goes: section 0 queries, 1 keys, 2 values; the two channels part ways only with an odd head size
  const int sec = c < Cq ? 0 : (c < Cq + Ck ? 1 : 2);
  const int in_sec = c - (sec == 0 ? 0 : (sec == 1 ? Cq : Cq + Ck));
  const int hs = sec == 2 ? Dv : D;                       // the head size of the section
  const int g = in_sec / hs, e = in_sec - g * hs;
  const bool together = two && e + 1 < hs && !(sec == 0 && c + 1 >= Cq) && !(sec == 1 && c + 1 >= Cq + Ck);
  const bool vec_store = together && (sec == 0 ? (Cq % 2 == 0) : (HD % 2 == 0 && e % 2 == 0));
  const int64_t plane_off = (int64_t)(sec == 2 ? nkv : 0) * page_size * HD + (int64_t)g * page_size * HD + e;   // inside a page
  const int64_t page_stride = (int64_t)2 * nkv * page_size * HD;
  double freq = 0.0;
  const bool rotated = rot > 0 && sec < 2 && e < rot && two;
  if (rotated && !angles) freq = inv_freq[e >> 1];
  const float* base = s.proj + c;
  pdl_wait();
  pdl_launch_dependents();
  float2 win[NT];                                          // u (bias included) at the last NT rows
  int win_end = -1;                                        // the global row after the newest one in ``win`` (-1: nothing held)
  const int t_end = min(T, (int)(blockIdx.x + 1) * tokens_a_thread);
  for (int t = blockIdx.x * tokens_a_thread; t < t_end; ++t) {
    const int b = token_req[t];
    const int tok0 = cu_seqlens[b], q_len = cu_seqlens[b + 1] - tok0;
    const int start = context_lens[b] - q_len;
    const int i = t - tok0;
    const int slot = state_slots[b];
    float y0, y1 = 0.f;
    if (TAPS >= 0 && two && i >= NT - 1) {
      // The usual case, all taps inside this step's rows of one request: no state, no start of the sequence.
      const bool slide = win_end == t && i >= NT;          // the rows t - NT .. t - 1 are held, and all are this request's
#pragma unroll
      for (int j = 0; j < NT - 1; ++j) {
        if (slide) {
          win[j] = win[j + 1];
        } else {
          const float* u = base + (int64_t)(t - (NT - 1 - j)) * s.stride;
          win[j] = vec2 ? *reinterpret_cast<const float2*>(u) : make_float2(u[0], u[1]);
          win[j].x += b0;
          win[j].y += b1;
        }
      }
      {
        const float* u = base + (int64_t)t * s.stride;
        win[NT - 1] = vec2 ? *reinterpret_cast<const float2*>(u) : make_float2(u[0], u[1]);
        win[NT - 1].x += b0;
        win[NT - 1].y += b1;
      }
      win_end = t + 1;
      if (TAPS == 0) {
        y0 = win[0].x;
        y1 = win[0].y;
      } else {
        y0 = 0.f;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          y0 = fmaf(w0[j], win[j].x, y0);
          y1 = fmaf(w1[j], win[j].y, y1);
        }
      }
    } else {
      win_end = -1;
      y0 = conv_output(s, wt, tok0, i, start, slot, c);
      if (two) y1 = conv_output(s, wt, tok0, i, start, slot, c + 1);
    }
    if (rotated) {
      float sn, cs;
      if (angles) {                                  // the step's table: (cosine, sine) per token and pair
        const float2 a = angles[(int64_t)t * (rot >> 1) + (e >> 1)];
        cs = a.x;
        sn = a.y;
      } else {
        rope_angle(positions[t], freq, &cs, &sn);
      }
      const float u = y0, v = y1;
      y0 = fmaf(u, cs, -v * sn);
      y1 = fmaf(v, cs, u * sn);
    }
    if (sec == 0 && together) {
      store_pair<TO>(q_out + (int64_t)t * Cq + c, y0, y1, vec_store);
    } else if (together) {
      const int where = slot_mapping ? slot_mapping[t] : -1;
      if (where >= 0) {
        const int page = where / page_size, off = where - page * page_size;
        store_pair<TO>(pool + page * page_stride + plane_off + (int64_t)off * HD, y0, y1, vec_store);
      }
    } else {
      // (an odd head size, or the last channel: each result finds its own place)
      const int where = slot_mapping ? slot_mapping[t] : -1;
      for (int k = 0; k < (two ? 2 : 1); ++k) {
        const int cc = c + k;
        const float y = k ? y1 : y0;
        if (cc < Cq) {
          q_out[(int64_t)t * Cq + cc] = from_f<TO>(y);
        } else if (where >= 0) {
          const int page = where / page_size, off = where - page * page_size;
          const int which = cc < Cq + Ck ? 0 : 1, rel = cc - (which ? Cq + Ck : Cq), h2 = which ? Dv : D;
          pool[((((int64_t)page * 2 + which) * nkv + rel / h2) * page_size + off) * HD + rel % h2] = from_f<TO>(y);
        }
      }
    }
    // A step in which every request brings one token: no other thread reads these channels of this slot, so the state
    // moves on here (rows up by one, the newest u last) and the second kernel is not launched.
    if (state_out && slot >= 0 && q_len == 1) {
      for (int cc = c; cc < c + (two ? 2 : 1); ++cc) {
        float* st = state_out + (int64_t)slot * (s.taps - 1) * s.C + cc;
        for (int k = 0; k < s.taps - 1; ++k) st[(int64_t)k * s.C] = conv_input(s, tok0, k - (s.taps - 2), start, slot, cc);
      }
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
// kernel.  angles: [T, rot/2] (cosine, sine) from me_rope_table, or null (each thread then forms its own).  q_out: [T, nh*D]; pool: [pages][2][nkv][page_size][HD] of out_dtype (unused without own_kv).
ME_API int me_conv_rope_kv(const float* proj, int64_t proj_stride, const float* bias, const float* wt, float* state, int taps,
                           const double* inv_freq, int rot, const int* positions, const int* token_req, const int* cu_seqlens,
                           const int* context_lens, const int* state_slots, const int* slot_mapping, void* q_out, void* pool,
                           int out_dtype, int T, int B, int nh, int nkv, int D, int Dv, int HD, int own_kv, int page_size,
                           int single_tokens, const float* angles, cudaStream_t stream) {
  if (T == 0) return 0;
  ME_REQUIRE(T > 0 && B > 0 && nh > 0 && D > 0 && taps >= 1, "me_conv_rope_kv: bad sizes");
  ME_REQUIRE(rot % 2 == 0 && rot >= 0 && rot <= D && (rot == 0 || D % 2 == 0), "me_conv_rope_kv: %d of %d elements rotated", rot, D);
  ME_REQUIRE(taps == 1 || (state != nullptr && wt != nullptr), "me_conv_rope_kv: %d taps need weights and a state", taps);
  ConvSrc s{proj, proj_stride, bias, state, nh * D + (own_kv ? nkv * (D + Dv) : 0), taps};
  const int threads = s.C >= 256 ? 256 : 64;
  const int per_thread = T >= 1024 ? CR_TOKENS : 1;
  dim3 grid((T + per_thread - 1) / per_thread, ((s.C + 1) / 2 + threads - 1) / threads);
  const int* sm = own_kv ? slot_mapping : (const int*)nullptr;
  float* st_out = (taps > 1 && single_tokens) ? state : (float*)nullptr;
  const int v2 = (proj_stride % 2 == 0 && ((uintptr_t)proj & 7) == 0) ? 1 : 0;
  const int kind = !wt ? 0 : (taps <= 4 ? taps : -1);      // which instance: the taps as a constant, or any number
#define ME_CR(TAPS_)                                                                                                         \
  ME_DISPATCH_DTYPE(out_dtype, TO,                                                                                           \
                    me_launch(conv_rope_kv_kernel<TO, TAPS_>, grid, dim3(threads), 0, stream, s, wt, inv_freq, rot, positions, \
                              token_req, cu_seqlens, context_lens, state_slots, sm, (TO*)q_out, (TO*)pool, nh, own_kv ? nkv : 0, \
                              D, Dv, HD, page_size, st_out, v2, T, (const float2*)angles, per_thread))
  switch (kind) {
    case 0: ME_CR(0); break;
    case 1: ME_CR(1); break;
    case 2: ME_CR(2); break;
    case 3: ME_CR(3); break;
    case 4: ME_CR(4); break;
    default: ME_CR(-1); break;
  }
#undef ME_CR
  ME_LAUNCH_CHECK("me_conv_rope_kv");
  if (taps > 1 && !single_tokens) {
    me_launch(conv_state_kernel, dim3(B, (s.C + threads - 1) / threads), dim3(threads), 0, stream, s, state, cu_seqlens,
              context_lens, state_slots);
    ME_LAUNCH_CHECK("me_conv_rope_kv (state)");
  }
  return 0;
}
