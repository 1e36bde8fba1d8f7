// The gated delta rule: a linear recurrence whose matrix state forgets per key channel and is corrected, not just
// added to, by every token; with the short causal convolutions that precede it.
//
//   convolution  y[t][c] = silu(sum_j w[c][j] x[t - taps + 1 + j][c])       inputs before a sequence's start are zero,
//                                                                           before this step's start they come from the state
//   unit vectors q = q / sqrt(sum q^2 + 1e-6) * q_scale ;  k = k / sqrt(sum k^2 + 1e-6)          per head
//   decay        g[i] = exp(-exp(A) softplus(a[i] + dt[i]))                 per head and key channel
//   step         S <- diag(g) S ;  u = beta (v - S^T k) ;  S <- S + k u^T ;  o = S^T q            beta = sigmoid(b)
//   out          = o / rms(o) * w * sigmoid(gate)                           per head, eps inside the root, w of size dv
//
// A block owns one head's S [d, dv] of one sequence in shared memory and walks the sequence's tokens of this step
// in order; thread j owns column j.  State, decay, beta, the unit vectors and the head norm are float32 whatever
// the run dtype.
#include "api.h"
#include "common.cuh"

namespace pe {

// ---- short convolution + silu -----------------------------------------------------------------------------------
// x: [n_tokens, ld] (channels at columns col0 .. col0 + channels), w: [channels, taps] float32,
// tail: [slots, taps - 1, channels] float32 (the last inputs of every sequence, oldest first).
template <typename T>
__global__ void short_conv_kernel(const T* x, long long ld, int col0, const float* __restrict__ w, int taps,
                                  const float* tail, const int* token_seq, const int* seq_slot, const int* seq_qstart,
                                  T* __restrict__ out, int n_tokens, int channels, int n_slots, int* status) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  if (t >= n_tokens) return;
  const int b = token_seq[t];
  const int first = seq_qstart[b];
  const int slot = seq_slot[b];
  if (slot < 0 || slot >= n_slots) {
    if (threadIdx.x == 0) report(status, kStatusSlotOutOfRange, t, slot, n_slots);
    return;
  }
  for (int c = threadIdx.x; c < channels; c += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int src = t - (taps - 1) + j;          // row of the step, if it belongs to this sequence
      float v;
      if (src >= first) v = to_f32<T>(x[(size_t)src * ld + col0 + c]);
      else v = tail[((size_t)slot * (taps - 1) + (taps - 1) - (first - src)) * channels + c];
      acc = fmaf(w[(size_t)c * taps + j], v, acc);
    }
    out[(size_t)t * channels + c] = from_f32<T>(acc / (1.f + expf(-acc)));
  }
}

// The new tail of every sequence: the last taps - 1 rows of (old tail, this step's inputs).  One thread per
// (sequence, channel) walks the rows oldest first, so a row is read before it is overwritten.
template <typename T>
__global__ void conv_tail_kernel(const T* x, long long ld, int col0, float* tail, int taps, const int* seq_slot,
                                 const int* seq_qstart, int n_seqs, int channels, int n_slots) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int b = blockIdx.y;
  const int slot = seq_slot[b];
  if (slot < 0 || slot >= n_slots) return;
  const int first = seq_qstart[b], len = seq_qstart[b + 1] - first, keep = taps - 1;
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < channels; c += gridDim.x * blockDim.x) {
    float* mine = tail + (size_t)slot * keep * channels + c;
    for (int r = 0; r < keep; ++r) {
      const int at = len + r;                      // index into (old tail, inputs)
      mine[(size_t)r * channels] = at < keep ? mine[(size_t)at * channels]
                                             : to_f32<T>(x[(size_t)(first + at - keep) * ld + col0 + c]);
    }
  }
}

// ---- the recurrence -----------------------------------------------------------------------------------------------
struct DeltaArgs {
  const void* qkv;          // [n_tokens, channels] after the convolution: q (kv_heads * d) | k (kv_heads * d) | v (heads * dv)
  const float* a;           // [n_tokens, heads * d]: the decay projection before its offset
  const float* dt_bias;     // [heads * d]
  const float* A_log;       // [heads]
  const float* b;           // [n_tokens, heads]: beta before the sigmoid
  const void* gate; long long gate_ld;   // [n_tokens, heads * dv] in the run dtype, before the sigmoid
  const float* norm_w;      // [dv]
  float eps, q_scale;
  void* out;                // [n_tokens, heads * dv]
  float* S;                 // [slots, heads, d, dv]
  const int* seq_slot; const int* seq_qstart;
  int n_seqs, heads, kv_heads, d, dv, n_slots;
  int* status;
};

template <typename T>
__global__ void delta_rule_kernel(DeltaArgs a) {
  extern __shared__ float sm[];
  __shared__ float red[32];
  const int d = a.d, dv = a.dv, head = blockIdx.x, b = blockIdx.y;
  const int kvh = head / (a.heads / a.kv_heads);
  float* S = sm;               // [d][dv]
  float* qs = S + (size_t)d * dv;
  float* ks = qs + d;
  float* gs = ks + d;
  pdl_wait_block();
  pdl_launch_dependents();
  const int slot = a.seq_slot[b];
  if (slot < 0 || slot >= a.n_slots) {
    if (threadIdx.x == 0 && head == 0) report(a.status, kStatusSlotOutOfRange, b, slot, a.n_slots);
    return;
  }
  const int t0 = a.seq_qstart[b], t1 = a.seq_qstart[b + 1];
  float* gS = a.S + ((size_t)slot * a.heads + head) * d * dv;
  for (int i = threadIdx.x; i < d * dv; i += blockDim.x) S[i] = gS[i];
  const int j = threadIdx.x;
  const int channels = 2 * a.kv_heads * d + a.heads * dv;
  const int k_col = a.kv_heads * d, v_col = 2 * a.kv_heads * d;
  const T* x = (const T*)a.qkv;
  const float rate = expf(a.A_log[head]);
  const float nw = j < dv ? a.norm_w[j] : 0.f;
  __syncthreads();
  for (int t = t0; t < t1; ++t) {
    float q2 = 0.f, k2 = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
      const float qq = to_f32<T>(x[(size_t)t * channels + kvh * d + i]);
      const float kk = to_f32<T>(x[(size_t)t * channels + k_col + kvh * d + i]);
      qs[i] = qq;
      ks[i] = kk;
      q2 += qq * qq;
      k2 += kk * kk;
      const float z = a.a[(size_t)t * a.heads * d + head * d + i] + a.dt_bias[head * d + i];
      const float softplus = z > 20.f ? z : log1pf(expf(z));
      gs[i] = expf(-rate * softplus);
    }
    q2 = block_sum(q2, red);
    k2 = block_sum(k2, red);
    const float qn = rsqrtf(q2 + 1e-6f) * a.q_scale, kn = rsqrtf(k2 + 1e-6f);
    const float beta = 1.f / (1.f + expf(-a.b[(size_t)t * a.heads + head]));
    float o = 0.f;
    if (j < dv) {
      float acc = 0.f;
      for (int i = 0; i < d; ++i) {
        const float s = gs[i] * S[(size_t)i * dv + j];
        S[(size_t)i * dv + j] = s;
        acc = fmaf(s, ks[i], acc);
      }
      const float u = beta * (to_f32<T>(x[(size_t)t * channels + v_col + head * dv + j]) - acc * kn);
      const float uk = u * kn;
      for (int i = 0; i < d; ++i) {
        const float s = fmaf(ks[i], uk, S[(size_t)i * dv + j]);
        S[(size_t)i * dv + j] = s;
        o = fmaf(s, qs[i], o);
      }
      o *= qn;
    }
    const float ss = block_sum(o * o, red);
    if (j < dv) {
      const float gate = to_f32<T>(((const T*)a.gate)[(size_t)t * a.gate_ld + head * dv + j]);
      const float y = o * rsqrtf(ss / (float)dv + a.eps) * nw / (1.f + expf(-gate));
      ((T*)a.out)[(size_t)t * a.heads * dv + head * dv + j] = from_f32<T>(y);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < d * dv; i += blockDim.x) gS[i] = S[i];
}

}  // namespace pe

extern "C" int pe_short_conv_silu(int dtype, const void* x, long long ld, int col0, const float* w, int taps, float* tail,
                                  const int* token_seq, const int* seq_slot, const int* seq_qstart, void* out,
                                  int n_tokens, int n_seqs, int channels, int n_slots, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return PE_OK;
  if (channels <= 0 || taps <= 0 || taps > 64 || col0 < 0 || col0 + channels > ld) return PE_ERR_BAD_ARGUMENT;
  const int threads = channels >= 1024 ? 256 : 128;
  if (dtype != PE_F32 && dtype != PE_BF16) return PE_ERR_UNSUPPORTED_DTYPE;
  if (dtype == PE_F32)
    pe::launch(pe::short_conv_kernel<float>, n_tokens, threads, 0, stream, (const float*)x, ld, col0, w, taps, (const float*)tail,
               token_seq, seq_slot, seq_qstart, (float*)out, n_tokens, channels, n_slots, status);
  else
    pe::launch(pe::short_conv_kernel<__nv_bfloat16>, n_tokens, threads, 0, stream, (const __nv_bfloat16*)x, ld, col0, w, taps,
               (const float*)tail, token_seq, seq_slot, seq_qstart, (__nv_bfloat16*)out, n_tokens, channels, n_slots, status);
  PE_LAUNCH_CHECK();
  if (taps > 1) {
    const dim3 grid((channels + 127) / 128, n_seqs);
    if (dtype == PE_F32)
      pe::launch(pe::conv_tail_kernel<float>, grid, dim3(128), 0, stream, (const float*)x, ld, col0, tail, taps, seq_slot,
                 seq_qstart, n_seqs, channels, n_slots);
    else
      pe::launch(pe::conv_tail_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, (const __nv_bfloat16*)x, ld, col0, tail, taps,
                 seq_slot, seq_qstart, n_seqs, channels, n_slots);
    PE_LAUNCH_CHECK();
  }
  return PE_OK;
}

extern "C" int pe_delta_rule_recurrence(int dtype, const void* qkv, const float* a, const float* dt_bias, const float* A_log,
                                        const float* b, const void* gate, long long gate_ld, const float* norm_w, float eps,
                                        float q_scale, void* out, float* S, const int* seq_slot, const int* seq_qstart,
                                        int n_seqs, int heads, int kv_heads, int d, int dv, int n_slots, int* status,
                                        cudaStream_t stream) {
  if (n_seqs <= 0) return PE_OK;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || d <= 0 || dv <= 0) return PE_ERR_BAD_ARGUMENT;
  const size_t smem = ((size_t)d * dv + 3 * (size_t)d) * sizeof(float);
  if (dv > 1024 || smem > 200 * 1024) return PE_ERR_UNSUPPORTED_SIZE;
  if (dtype != PE_F32 && dtype != PE_BF16) return PE_ERR_UNSUPPORTED_DTYPE;
  pe::DeltaArgs args{qkv, a, dt_bias, A_log, b, gate, gate_ld, norm_w, eps, q_scale, out, S, seq_slot, seq_qstart,
                     n_seqs, heads, kv_heads, d, dv, n_slots, status};
  const int widest = dv > d ? dv : d;
  const int threads = (widest + 31) / 32 * 32 > 1024 ? 1024 : (widest + 31) / 32 * 32;
  auto kernel = dtype == PE_F32 ? pe::delta_rule_kernel<float> : pe::delta_rule_kernel<__nv_bfloat16>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  pe::launch(kernel, dim3(heads, n_seqs), dim3(threads), smem, stream, args);
  PE_LAUNCH_CHECK();
  return PE_OK;
}
