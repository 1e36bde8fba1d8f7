// A matrix-memory recurrence with exponential gates and a running maximum (the mLSTM cell of xLSTM), for prompts and
// for single tokens alike.
//
//   gates     i[t] = cap tanh((gi[t] + bi) / cap)          f[t] = logsigmoid(cap tanh((gf[t] + bf) / cap))
//   maximum   m'   = max(f + m, i)                          m starts at 0
//   update    S'   = e^(f + m - m') S + e^(i - m') k v^T    n' = e^(f + m - m') n + e^(i - m') k
//   read      o    = S'^T q / (max(|n' . q|, e^(-m')) + 1e-6)     q already carries its factor d^(-1/2)
//   out       = o / rms(o) * w * sigmoid(g)                 per head, eps inside the root
//
// A block owns one head's S [d, dv], n [d] and m of one sequence in shared memory and walks the sequence's tokens
// of this step in order; thread j owns column j of S.  Gates, state, the read's denominator and the head norm are
// float32 whatever the run dtype; q, k, v, g come from matrix products in the run dtype, the two gate
// pre-activations from a product that writes float32.
#include "api.h"
#include "common.cuh"

namespace pe {

struct MlstmArgs {
  const void* q; const void* k; const void* v; const void* g;   // rows of the run dtype, `ld` elements apart
  long long ld;
  const float* gates;     // [n_tokens, 2 * heads]: input-gate pre-activations, then forget-gate ones
  const float* gate_bias; // [2 * heads]
  const float* norm_w;    // [heads * dv]
  float cap, eps, q_scale;
  void* out;              // [n_tokens, heads * dv] in the run dtype
  float* S;               // [slots, heads, d, dv]
  float* n;               // [slots, heads, d]
  float* m;               // [slots, heads]
  const int* seq_slot; const int* seq_qstart;
  int n_seqs, heads, d, dv, n_slots;
  int* status;
};

__device__ __forceinline__ float log_sigmoid(float z) {
  // log(1 / (1 + e^-z)) without overflow on either side
  return fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
}

template <typename T>
__global__ void mlstm_kernel(MlstmArgs a) {
  extern __shared__ float sm[];
  __shared__ float red[32];
  const int d = a.d, dv = a.dv, head = blockIdx.x, b = blockIdx.y;
  float* S = sm;                  // [d][dv]
  float* nvec = S + (size_t)d * dv;
  float* qs = nvec + d;
  float* ks = qs + d;
  pdl_wait_block();
  pdl_launch_dependents();
  const int slot = a.seq_slot[b];
  if (slot < 0 || slot >= a.n_slots) {
    if (threadIdx.x == 0 && head == 0) report(a.status, kStatusSlotOutOfRange, b, slot, a.n_slots);
    return;
  }
  const int t0 = a.seq_qstart[b], t1 = a.seq_qstart[b + 1];
  float* gS = a.S + ((size_t)slot * a.heads + head) * d * dv;
  float* gn = a.n + ((size_t)slot * a.heads + head) * d;
  for (int i = threadIdx.x; i < d * dv; i += blockDim.x) S[i] = gS[i];
  for (int i = threadIdx.x; i < d; i += blockDim.x) nvec[i] = gn[i];
  float m = a.m[(size_t)slot * a.heads + head];
  const int j = threadIdx.x;
  const float bi = a.gate_bias[head], bf = a.gate_bias[a.heads + head];
  const T* q = (const T*)a.q; const T* k = (const T*)a.k; const T* v = (const T*)a.v; const T* g = (const T*)a.g;
  __syncthreads();
  for (int t = t0; t < t1; ++t) {
    const float gi = a.cap * tanhf((a.gates[(size_t)t * 2 * a.heads + head] + bi) / a.cap);
    const float gf = log_sigmoid(a.cap * tanhf((a.gates[(size_t)t * 2 * a.heads + a.heads + head] + bf) / a.cap));
    const float m_new = fmaxf(gf + m, gi);
    const float keep = expf(gf + m - m_new), take = expf(gi - m_new);
    m = m_new;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
      const float kk = to_f32<T>(k[(size_t)t * a.ld + head * d + i]);
      qs[i] = to_f32<T>(q[(size_t)t * a.ld + head * d + i]) * a.q_scale;
      ks[i] = kk;
      nvec[i] = keep * nvec[i] + take * kk;
    }
    __syncthreads();
    float o = 0.f;
    if (j < dv) {
      const float tv = take * to_f32<T>(v[(size_t)t * a.ld + head * dv + j]);
      float acc = 0.f, nq = 0.f;
      for (int i = 0; i < d; ++i) {
        const float s = fmaf(keep, S[(size_t)i * dv + j], ks[i] * tv);
        S[(size_t)i * dv + j] = s;
        acc = fmaf(s, qs[i], acc);
        nq = fmaf(nvec[i], qs[i], nq);
      }
      o = acc / (fmaxf(fabsf(nq), expf(-m)) + 1e-6f);
    }
    const float ss = block_sum(o * o, red);   // its barriers also order this token's reads of q, k before the next writes
    if (j < dv) {
      const float gate = to_f32<T>(g[(size_t)t * a.ld + head * dv + j]);
      const float y = o * rsqrtf(ss / (float)dv + a.eps) * a.norm_w[head * dv + j] / (1.f + expf(-gate));
      ((T*)a.out)[(size_t)t * a.heads * dv + head * dv + j] = from_f32<T>(y);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < d * dv; i += blockDim.x) gS[i] = S[i];
  for (int i = threadIdx.x; i < d; i += blockDim.x) gn[i] = nvec[i];
  if (threadIdx.x == 0) a.m[(size_t)slot * a.heads + head] = m;
}

}  // namespace pe

extern "C" int pe_mlstm_recurrence(int dtype, const void* q, const void* k, const void* v, const void* g, long long ld,
                                   const float* gates, const float* gate_bias, const float* norm_w, float cap, float eps,
                                   float q_scale, void* out, float* S, float* n, float* m, const int* seq_slot,
                                   const int* seq_qstart, int n_seqs, int heads, int d, int dv, int n_slots, int* status,
                                   cudaStream_t stream) {
  if (n_seqs <= 0) return PE_OK;
  if (heads <= 0 || d <= 0 || dv <= 0 || !(cap > 0.f)) return PE_ERR_BAD_ARGUMENT;
  const size_t smem = ((size_t)d * dv + 3 * (size_t)d) * sizeof(float);
  if (dv > 1024 || smem > 200 * 1024) return PE_ERR_UNSUPPORTED_SIZE;
  pe::MlstmArgs a{q, k, v, g, ld, gates, gate_bias, norm_w, cap, eps, q_scale, out, S, n, m, seq_slot, seq_qstart,
                  n_seqs, heads, d, dv, n_slots, status};
  const int threads = ((dv > d ? dv : d) + 31) / 32 * 32 > 1024 ? 1024 : ((dv > d ? dv : d) + 31) / 32 * 32;
  auto kernel = dtype == PE_F32 ? pe::mlstm_kernel<float> : pe::mlstm_kernel<__nv_bfloat16>;
  if (dtype != PE_F32 && dtype != PE_BF16) return PE_ERR_UNSUPPORTED_DTYPE;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  pe::launch(kernel, dim3(heads, n_seqs), dim3(threads), smem, stream, a);
  PE_LAUNCH_CHECK();
  return PE_OK;
}
