// The middle of a layer's token input: g[t, j] = gelu_tanh(z[t, j]) * table[token_t, first + j], where z is the product of
// the stream with the layer's gate matrix and ``table`` a second embedding of which every layer has a slice of ``dim``
// columns.  gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))).  A token id ~j stands for feedback[j].
#include "common.cuh"

template <typename TZ, typename TE, typename TO>
__global__ void __launch_bounds__(128)
token_side_gate_kernel(const TZ* __restrict__ z, int64_t z_stride, const int* __restrict__ ids, const int* __restrict__ feedback,
                       const TE* __restrict__ table, int64_t table_stride, int vocab, int first, int dim, TO* __restrict__ out) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 && feedback) id = feedback[~id];
  if (id < 0 || id >= vocab) id = 0;           // the embedding kernel has flagged it
  for (int j = threadIdx.x; j < dim; j += blockDim.x) {
    const float v = to_f<TZ>(z[(int64_t)t * z_stride + j]);
    const float gelu = 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    out[(int64_t)t * dim + j] = from_f<TO>(gelu * to_f<TE>(table[(int64_t)id * table_stride + first + j]));
  }
}

ME_API int me_token_side_gate(const void* z, int z_dtype, int64_t z_stride, const int* ids, const int* feedback, const void* table,
                              int table_dtype, int64_t table_stride, int vocab, int first, int dim, void* out, int out_dtype, int T,
                              cudaStream_t stream) {
  if (T == 0) return 0;
  ME_REQUIRE(dim > 0 && first >= 0 && first + dim <= table_stride, "me_token_side_gate: slice [%d, %d) of %lld columns", first,
             first + dim, (long long)table_stride);
  ME_DISPATCH_DTYPE(z_dtype, TZ, ME_DISPATCH_DTYPE(table_dtype, TE, ME_DISPATCH_DTYPE(out_dtype, TO,
      me_launch(token_side_gate_kernel<TZ, TE, TO>, dim3(T), dim3(128), 0, stream, (const TZ*)z, z_stride, ids, feedback,
                (const TE*)table, table_stride, vocab, first, dim, (TO*)out))));
  ME_LAUNCH_CHECK("me_token_side_gate");
  return 0;
}
