// PolyNorm activation over a token's vector z of F values:
//   out = a N(z) + b N(z^2) + c N(z^3) + e,   N(v) = v / sqrt(mean(v^2) + eps),
// powers taken element by element.  The three mean squares are mean(z^2), mean(z^4), mean(z^6); sums and
// factors are float32, the result is rounded once to the output's dtype.
#include "common.cuh"

template <typename TZ, typename TO>
__global__ void __launch_bounds__(256)
polynorm_kernel(const TZ* __restrict__ z, int64_t ldz, const float* __restrict__ coef, float eps, TO* __restrict__ out,
                int64_t ldo, int F) {
  __shared__ float red[32];
  const float a = coef[0], b = coef[1], c = coef[2], e = coef[3];
  pdl_wait();
  pdl_launch_dependents();
  const TZ* zr = z + (int64_t)blockIdx.x * ldz;
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
  for (int f = threadIdx.x; f < F; f += blockDim.x) {
    const float v = to_f<TZ>(zr[f]), v2 = v * v;
    s2 += v2;
    s4 = fmaf(v2, v2, s4);
    s6 = fmaf(v2 * v, v2 * v, s6);
  }
  const float r1 = 1.0f / sqrtf(block_sum(s2, red) / (float)F + eps);
  const float r2 = 1.0f / sqrtf(block_sum(s4, red) / (float)F + eps);
  const float r3 = 1.0f / sqrtf(block_sum(s6, red) / (float)F + eps);
  TO* o = out + (int64_t)blockIdx.x * ldo;
  for (int f = threadIdx.x; f < F; f += blockDim.x) {
    const float v = to_f<TZ>(zr[f]), v2 = v * v;
    o[f] = from_f<TO>(a * (v * r1) + b * (v2 * r2) + c * (v2 * v * r3) + e);
  }
}

ME_API int me_polynorm(const void* z, int z_dtype, int64_t ldz, const float* coef, float eps, void* out, int out_dtype,
                       int64_t ldo, int T, int F, cudaStream_t stream) {
  if (T == 0) return 0;
  ME_REQUIRE(T > 0 && F > 0, "me_polynorm: bad sizes T=%d F=%d", T, F);
  const int threads = F >= 1024 ? 256 : 128;
  ME_DISPATCH_DTYPE(z_dtype, TZ, ME_DISPATCH_DTYPE(out_dtype, TO,
      me_launch(polynorm_kernel<TZ, TO>, dim3(T), dim3(threads), 0, stream, (const TZ*)z, ldz, coef, eps, (TO*)out, ldo, F)));
  ME_LAUNCH_CHECK("me_polynorm");
  return 0;
}
