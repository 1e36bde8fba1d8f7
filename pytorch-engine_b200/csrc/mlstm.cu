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
  int chunk;              // tokens per chunk (modes 1 and 3), 0: the whole step in one go
  int max_chunks;
  float* scratch;         // [n_seqs, max_chunks, heads, d * dv + d + 3]: S, n, then the chunk's own maximum, its summed
                          // forget gates, and the maximum at its start
  int* status;
};

__device__ __forceinline__ float log_sigmoid(float z) {
  // log(1 / (1 + e^-z)) without overflow on either side
  return fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
}

__host__ __device__ inline size_t mlstm_unit(int d, int dv) { return (size_t)d * dv + d + 3; }

// MODE 0: the whole step: start from the slot's state, write outputs, write the state back.
// MODE 1: chunk blockIdx.z from an empty state (S = 0, n = 0, maximum -inf): leaves its end state, its own maximum and
//         the sum of its forget gates; no outputs.  The update is linear in (S, n), so the chain kernel can put the true
//         start in front of it: with F the sum of the chunk's forget gates and M its own maximum,
//         m' = max(F + m, M);  S' = e^(F + m - m') S + e^(M - m') S_chunk   (n likewise).
// MODE 3: chunk blockIdx.z from its true start (as the chain kernel left it): writes outputs; the sequence's last chunk
//         writes the state back.
// DREG > 0: d <= DREG and thread j keeps its column of S in registers; DREG == 0: S lives in shared memory.
template <typename T, int MODE, int DREG>
__global__ void __launch_bounds__(DREG == 128 ? 256 : (DREG == 64 ? 512 : 1024)) mlstm_kernel(MlstmArgs a) {
  extern __shared__ float sm[];
  __shared__ float red[32];
  const int d = a.d, dv = a.dv, head = blockIdx.x, b = blockIdx.y, c = blockIdx.z;
  constexpr int DP = DREG > 0 ? DREG : 1;
  const int dpad = DREG > 0 ? DREG : d;            // vectors are padded with zeros up to the register tile
  float* S = sm;                                   // [d][dv] (DREG == 0 only)
  float* nvec = S + (DREG > 0 ? 0 : (size_t)d * dv);
  float* qs = nvec + dpad;
  float* ks = qs + dpad;
  pdl_wait_block();
  pdl_launch_dependents();
  const int slot = a.seq_slot[b];
  if (slot < 0 || slot >= a.n_slots) {
    if (threadIdx.x == 0 && head == 0 && c == 0) report(a.status, kStatusSlotOutOfRange, b, slot, a.n_slots);
    return;
  }
  const int q0 = a.seq_qstart[b], q1 = a.seq_qstart[b + 1];
  int t0 = q0, t1 = q1;
  if (MODE != 0) {
    t0 = q0 + c * a.chunk;
    t1 = min(q1, t0 + a.chunk);
    if (t0 >= q1) return;
    if (MODE == 1 && t1 == q1) return;             // nothing follows the sequence's last chunk
  }
  const size_t unit = mlstm_unit(d, dv);
  float* cs = MODE != 0 ? a.scratch + (((size_t)b * a.max_chunks + c) * a.heads + head) * unit : nullptr;
  float* gS = a.S + ((size_t)slot * a.heads + head) * d * dv;
  float* gn = a.n + ((size_t)slot * a.heads + head) * d;
  const float* src_S = MODE == 0 ? gS : cs;
  const float* src_n = MODE == 0 ? gn : cs + (size_t)d * dv;
  const int j = threadIdx.x;
  float Sr[DP];
  float m;
  if (MODE == 1) {
    if (DREG > 0) {
#pragma unroll
      for (int i = 0; i < DP; ++i) Sr[i] = 0.f;
    } else {
      for (int i = threadIdx.x; i < d * dv; i += blockDim.x) S[i] = 0.f;
    }
    for (int i = threadIdx.x; i < dpad; i += blockDim.x) nvec[i] = 0.f;
    m = -INFINITY;
  } else {
    if (DREG > 0) {
#pragma unroll
      for (int i = 0; i < DP; ++i) Sr[i] = (i < d && j < dv) ? src_S[(size_t)i * dv + j] : 0.f;
    } else {
      for (int i = threadIdx.x; i < d * dv; i += blockDim.x) S[i] = src_S[i];
    }
    for (int i = threadIdx.x; i < dpad; i += blockDim.x) nvec[i] = i < d ? src_n[i] : 0.f;
    m = MODE == 0 ? a.m[(size_t)slot * a.heads + head] : cs[unit - 1];
  }
  for (int i = d + threadIdx.x; i < dpad; i += blockDim.x) qs[i] = ks[i] = 0.f;
  float fsum = 0.f;
  const float bi = a.gate_bias[head], bf = a.gate_bias[a.heads + head];
  const T* q = (const T*)a.q; const T* k = (const T*)a.k; const T* v = (const T*)a.v; const T* g = (const T*)a.g;
  __syncthreads();
  for (int t = t0; t < t1; ++t) {
    const float gi = a.cap * tanhf((a.gates[(size_t)t * 2 * a.heads + head] + bi) / a.cap);
    const float gf = log_sigmoid(a.cap * tanhf((a.gates[(size_t)t * 2 * a.heads + a.heads + head] + bf) / a.cap));
    const float m_new = fmaxf(gf + m, gi);
    const float keep = expf(gf + m - m_new), take = expf(gi - m_new);
    m = m_new;
    fsum += gf;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
      const float kk = to_f32<T>(k[(size_t)t * a.ld + head * d + i]);
      if (MODE != 1) qs[i] = to_f32<T>(q[(size_t)t * a.ld + head * d + i]) * a.q_scale;
      ks[i] = kk;
      nvec[i] = keep * nvec[i] + take * kk;
    }
    __syncthreads();
    float o = 0.f;
    if (j < dv) {
      const float tv = take * to_f32<T>(v[(size_t)t * a.ld + head * dv + j]);
      float acc = 0.f, nq = 0.f;
      if (DREG > 0) {
#pragma unroll
        for (int i = 0; i < DP; i += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(ks + i);
#pragma unroll
          for (int e = 0; e < 4; ++e) Sr[i + e] = fmaf(keep, Sr[i + e], (&k4.x)[e] * tv);
          if (MODE != 1) {
            const float4 q4 = *reinterpret_cast<const float4*>(qs + i);
            const float4 n4 = *reinterpret_cast<const float4*>(nvec + i);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              acc = fmaf(Sr[i + e], (&q4.x)[e], acc);
              nq = fmaf((&n4.x)[e], (&q4.x)[e], nq);
            }
          }
        }
      } else {
        for (int i = 0; i < d; ++i) {
          const float s = fmaf(keep, S[(size_t)i * dv + j], ks[i] * tv);
          S[(size_t)i * dv + j] = s;
          if (MODE != 1) {
            acc = fmaf(s, qs[i], acc);
            nq = fmaf(nvec[i], qs[i], nq);
          }
        }
      }
      o = acc / (fmaxf(fabsf(nq), expf(-m)) + 1e-6f);
    }
    if (MODE == 1) {
      __syncthreads();                           // this token's k has been read before the next one is written
      continue;
    }
    const float ss = block_sum(o * o, red);   // its barriers also order this token's reads of q, k before the next writes
    if (j < dv) {
      const float gate = to_f32<T>(g[(size_t)t * a.ld + head * dv + j]);
      const float y = o * rsqrtf(ss / (float)dv + a.eps) * a.norm_w[head * dv + j] / (1.f + expf(-gate));
      ((T*)a.out)[(size_t)t * a.heads * dv + head * dv + j] = from_f32<T>(y);
    }
  }
  __syncthreads();
  if (MODE == 3 && t1 != q1) return;               // only the sequence's last chunk leaves the state
  float* dst_S = MODE == 1 ? cs : gS;
  float* dst_n = MODE == 1 ? cs + (size_t)d * dv : gn;
  if (DREG > 0) {
    if (j < dv) {
#pragma unroll
      for (int i = 0; i < DP; ++i)
        if (i < d) dst_S[(size_t)i * dv + j] = Sr[i];
    }
  } else {
    for (int i = threadIdx.x; i < d * dv; i += blockDim.x) dst_S[i] = S[i];
  }
  for (int i = threadIdx.x; i < d; i += blockDim.x) dst_n[i] = nvec[i];
  if (threadIdx.x == 0) {
    if (MODE == 1) {
      cs[unit - 3] = m;
      cs[unit - 2] = fsum;
    } else {
      a.m[(size_t)slot * a.heads + head] = m;
    }
  }
}

// Chain the chunks: on entry scratch[c] holds chunk c's end state from an empty start (every chunk but the sequence's
// last); on exit it holds chunk c's true start state, chunk 0's being the slot's state.  One thread per element of
// (S, n); every thread follows the scalar chain of maxima itself.
__global__ void mlstm_chain_kernel(MlstmArgs a) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int head = blockIdx.x, b = blockIdx.y, d = a.d, dv = a.dv;
  const int e = blockIdx.z * blockDim.x + threadIdx.x;
  const int elems = d * dv + d;
  const int slot = a.seq_slot[b];
  if (slot < 0 || slot >= a.n_slots || e >= elems) return;
  const int q_len = a.seq_qstart[b + 1] - a.seq_qstart[b];
  const int n_chunks = (q_len + a.chunk - 1) / a.chunk;
  const size_t unit = mlstm_unit(d, dv);
  float* cs = a.scratch + ((size_t)b * a.max_chunks * a.heads + head) * unit;   // chunk c: cs + c * per
  const size_t per = (size_t)a.heads * unit;
  float cur = e < d * dv ? a.S[((size_t)slot * a.heads + head) * d * dv + e] : a.n[((size_t)slot * a.heads + head) * d + (e - d * dv)];
  float m = a.m[(size_t)slot * a.heads + head];
  for (int c = 0; c < n_chunks; ++c) {
    float* u = cs + (size_t)c * per;
    const bool has = c + 1 < n_chunks;
    const float loc = has ? u[e] : 0.f, M = has ? u[unit - 3] : 0.f, F = has ? u[unit - 2] : 0.f;
    u[e] = cur;
    if (e == 0) u[unit - 1] = m;
    if (has) {
      const float m_new = fmaxf(F + m, M);
      cur = expf(F + m - m_new) * cur + expf(M - m_new) * loc;
      m = m_new;
    }
  }
}

template <typename T, int DREG>
static int mlstm_run(const MlstmArgs& a, int max_q, cudaStream_t stream) {
  const int d = a.d, dv = a.dv;
  const int dpad = DREG > 0 ? DREG : d;
  const size_t smem = ((DREG > 0 ? 0 : (size_t)d * dv) + 3 * (size_t)dpad) * sizeof(float);
  const int widest = dv > d ? dv : d;
  int threads = (widest + 31) / 32 * 32;
  const int cap_threads = DREG == 128 ? 256 : (DREG == 64 ? 512 : 1024);
  if (threads > cap_threads) threads = cap_threads;
  if (DREG > 0 && dv > threads) return PE_ERR_UNSUPPORTED_SIZE;
  auto k0 = mlstm_kernel<T, 0, DREG>;
  auto k1 = mlstm_kernel<T, 1, DREG>;
  auto k3 = mlstm_kernel<T, 3, DREG>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(k0, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k3, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  if (a.chunk > 0) {
    const dim3 grid(a.heads, a.n_seqs, a.max_chunks);
    launch(k1, grid, dim3(threads), smem, stream, a);
    const int elems = d * dv + d;
    launch(mlstm_chain_kernel, dim3(a.heads, a.n_seqs, (elems + 255) / 256), dim3(256), 0, stream, a);
    launch(k3, grid, dim3(threads), smem, stream, a);
  } else {
    launch(k0, dim3(a.heads, a.n_seqs, 1), dim3(threads), smem, stream, a);
  }
  (void)max_q;
  return PE_OK;
}

}  // namespace pe

// Floats of scratch that the chunked form needs for `max_chunks` chunks per sequence.
extern "C" long long pe_mlstm_scratch_floats(int n_seqs, int heads, int d, int dv, int max_chunks) {
  return (long long)n_seqs * max_chunks * heads * (long long)pe::mlstm_unit(d, dv);
}

// chunk > 0: prompts cut into chunks of that many tokens (scratch from pe_mlstm_scratch_floats, max_chunks >=
// ceil(max_q / chunk)); chunk == 0: each sequence's tokens in one go (single tokens, short prompts).
extern "C" int pe_mlstm_recurrence(int dtype, const void* q, const void* k, const void* v, const void* g, long long ld,
                                   const float* gates, const float* gate_bias, const float* norm_w, float cap, float eps,
                                   float q_scale, void* out, float* S, float* n, float* m, const int* seq_slot,
                                   const int* seq_qstart, int n_seqs, int max_q, int heads, int d, int dv, int n_slots,
                                   int chunk, int max_chunks, float* scratch, int* status, cudaStream_t stream) {
  if (n_seqs <= 0) return PE_OK;
  if (heads <= 0 || d <= 0 || dv <= 0 || !(cap > 0.f)) return PE_ERR_BAD_ARGUMENT;
  if (dv > 1024) return PE_ERR_UNSUPPORTED_SIZE;
  if (dtype != PE_F32 && dtype != PE_BF16) return PE_ERR_UNSUPPORTED_DTYPE;
  pe::MlstmArgs a{q, k, v, g, ld, gates, gate_bias, norm_w, cap, eps, q_scale, out, S, n, m, seq_slot, seq_qstart,
                  n_seqs, heads, d, dv, n_slots, 0, 1, nullptr, status};
  if (chunk > 0) {
    if (!scratch || max_chunks <= 0 || (long long)max_chunks * chunk < max_q || max_chunks > 65535) return PE_ERR_BAD_ARGUMENT;
    a.chunk = chunk; a.max_chunks = max_chunks; a.scratch = scratch;
  }
  // the state's columns in registers where a column fits (key sizes up to 128, value sizes up to the block), in shared
  // memory otherwise
  const int reg = (d <= 32) ? 32 : (d <= 64 && dv <= 512 ? 64 : (d <= 128 && dv <= 256 ? 128 : 0));
  if (reg == 0 && ((size_t)d * dv + 3 * (size_t)d) * sizeof(float) > 200 * 1024) return PE_ERR_UNSUPPORTED_SIZE;
  int rc;
#define PE_MLSTM(T)                                                          \
  (reg == 32 ? pe::mlstm_run<T, 32>(a, max_q, stream)                        \
   : reg == 64 ? pe::mlstm_run<T, 64>(a, max_q, stream)                      \
   : reg == 128 ? pe::mlstm_run<T, 128>(a, max_q, stream) : pe::mlstm_run<T, 0>(a, max_q, stream))
  rc = dtype == PE_F32 ? PE_MLSTM(float) : PE_MLSTM(__nv_bfloat16);
#undef PE_MLSTM
  if (rc != PE_OK) return rc;
  PE_LAUNCH_CHECK();
  return PE_OK;
}
