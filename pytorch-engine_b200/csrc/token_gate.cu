// A gate on a per-token table entry: out[t] = gelu_tanh(gx[t]) * table[token[t], col0 : col0 + dim].
// gx is a small projection of the residual stream; the table row belongs to the token itself (a second,
// narrow embedding of which every layer reads its own columns).  gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2/pi)
// (z + 0.044715 z^3))), in float32.
#include "api.h"
#include "common.cuh"

namespace pe {

template <typename T>
__global__ void token_gate_kernel(const T* gx, const T* __restrict__ table, long long table_ld, int col0, const int* tokens,
                                  T* __restrict__ out, int n_tokens, int dim, int vocab, int* status) {
  pdl_wait_block();
  pdl_launch_dependents();
  const size_t total = (size_t)n_tokens * dim;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int t = (int)(i / dim), c = (int)(i - (size_t)t * dim);
    const int id = tokens[t];
    if (id < 0 || id >= vocab) {
      if (c == 0) report(status, kStatusTokenOutOfRange, t, id, vocab);
      out[i] = from_f32<T>(0.f);
      continue;
    }
    const float z = to_f32<T>(gx[i]);
    const float e = to_f32<T>(table[(size_t)id * table_ld + col0 + c]);
    const float gelu = 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    out[i] = from_f32<T>(gelu * e);
  }
}

}  // namespace pe

extern "C" int pe_token_gate(int dtype, const void* gx, const void* table, long long table_ld, int col0, const int* tokens,
                             void* out, int n_tokens, int dim, int vocab, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return PE_OK;
  if (dim <= 0 || vocab <= 0 || col0 < 0 || col0 + dim > table_ld) return PE_ERR_BAD_ARGUMENT;
  const size_t total = (size_t)n_tokens * dim;
  const int threads = 256;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > pe::kSMs * 16) blocks = pe::kSMs * 16;
  if (dtype == PE_F32)
    pe::launch(pe::token_gate_kernel<float>, (int)blocks, threads, 0, stream, (const float*)gx, (const float*)table, table_ld, col0,
               tokens, (float*)out, n_tokens, dim, vocab, status);
  else if (dtype == PE_BF16)
    pe::launch(pe::token_gate_kernel<__nv_bfloat16>, (int)blocks, threads, 0, stream, (const __nv_bfloat16*)gx,
               (const __nv_bfloat16*)table, table_ld, col0, tokens, (__nv_bfloat16*)out, n_tokens, dim, vocab, status);
  else
    return PE_ERR_UNSUPPORTED_DTYPE;
  PE_LAUNCH_CHECK();
  return PE_OK;
}
