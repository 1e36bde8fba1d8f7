// A matrix-memory recurrence with exponential gates and a running maximum (the mLSTM cell of xLSTM), for prompts and
// for single tokens alike.
//
//   gates     i[t] = cap tanh((gi[t] + bi) / cap)          f[t] = logsigmoid(cap tanh((gf[t] + bf) / cap))
//   maximum   m'   = max(f + m, i)                          m starts at 0
//   update    S'   = e^(f + m - m') S + e^(i - m') k v^T    n' = e^(f + m - m') n + e^(i - m') k
//   read      o    = S'^T q / (max(|n' . q|, e^(-m')) + 1e-6)     q already carries its factor d^(-1/2)
//   out       = o / rms(o) * w * sigmoid(g)                 per head, eps inside the root
//
// A block owns one head's S [d, dv], n [d] and m of one sequence (S in registers or in shared memory) and walks the
// sequence's tokens of this step in order; thread j owns column j of S.  Gates, state, the read's denominator and the head norm are
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
//
// Tokens are taken `batch` at a time: their k, q, v, g rows are staged in shared memory with all loads in flight at
// once, their gates are computed side by side, and one thread runs the chain of maxima over the batch; the walk over
// the batch's tokens then reads shared memory only (a walk that loads each token's rows when it gets there spends most
// of its time waiting for them).
constexpr int kMlstmBatch = 32;

template <typename T>
__host__ __device__ inline size_t mlstm_smem_bytes(int d, int dv, int dreg, int batch) {
  const size_t dpad = dreg > 0 ? dreg : d;       // dreg: the padded key size of a register variant
  return ((dreg > 0 ? 0 : (size_t)d * dv) + dpad + 2 * (size_t)batch * dpad) * sizeof(float) + 2 * (size_t)batch * dv * sizeof(T);
}

// SPLIT == 2 (with DREG == 128): two threads share a column, each with 64 of its rows in registers; they are lanes l and
// l ^ 16 of one warp and add their partial sums with one shuffle.  Half the registers a thread, so four times the
// warps an SM holds: the walk waits on shared-memory and arithmetic latencies, which more warps hide.
template <typename T, int MODE, int DREG, int SPLIT>
__global__ void __launch_bounds__(DREG == 64 ? 512 : 1024) mlstm_kernel(MlstmArgs a, int batch) {
  extern __shared__ __align__(16) float sm[];
  __shared__ float red[32];
  __shared__ float s_keep[kMlstmBatch], s_take[kMlstmBatch], s_em[kMlstmBatch];
  const int d = a.d, dv = a.dv, head = blockIdx.x, b = blockIdx.y, c = blockIdx.z;
  constexpr int DP = DREG > 0 ? DREG : 1;          // rows of a column that a thread keeps
  const int dpad = DREG > 0 ? DREG * SPLIT : d;    // vectors are padded with zeros up to the register tile
  float* S = sm;                                   // [d][dv] (DREG == 0 only)
  float* nvec = S + (DREG > 0 ? 0 : (size_t)d * dv);
  float* kb = nvec + dpad;                         // [batch][dpad]
  float* qb = kb + (size_t)batch * dpad;           // [batch][dpad]
  T* vb = reinterpret_cast<T*>(qb + (size_t)batch * dpad);   // [batch][dv]
  T* gb = vb + (size_t)batch * dv;                 // [batch][dv]
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
  // the thread's column and, with two threads a column, the first of its rows
  const int j = SPLIT == 2 ? (threadIdx.x >> 5) * 16 + (threadIdx.x & 15) : threadIdx.x;
  const int i0 = SPLIT == 2 ? ((threadIdx.x >> 4) & 1) * DP : 0;
  float Sr[DP];
  float m;                                         // followed by thread 0
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
      for (int i = 0; i < DP; ++i) Sr[i] = (i0 + i < d && j < dv) ? src_S[(size_t)(i0 + i) * dv + j] : 0.f;
    } else {
      for (int i = threadIdx.x; i < d * dv; i += blockDim.x) S[i] = src_S[i];
    }
    for (int i = threadIdx.x; i < dpad; i += blockDim.x) nvec[i] = i < d ? src_n[i] : 0.f;
    m = MODE == 0 ? a.m[(size_t)slot * a.heads + head] : cs[unit - 1];
  }
  if (dpad > d)
    for (int e = threadIdx.x; e < batch * (dpad - d); e += blockDim.x) {
      const int tt = e / (dpad - d), i = d + e % (dpad - d);
      kb[(size_t)tt * dpad + i] = 0.f;
      qb[(size_t)tt * dpad + i] = 0.f;
    }
  float fsum = 0.f;
  const float bi = a.gate_bias[head], bf = a.gate_bias[a.heads + head];
  const float nw = (MODE != 1 && j < dv) ? a.norm_w[head * dv + j] : 0.f;
  const T* q = (const T*)a.q; const T* k = (const T*)a.k; const T* v = (const T*)a.v; const T* g = (const T*)a.g;
  // 16-byte staging where the rows allow it (a token's rows keep their alignment from token to token)
  const bool smem_ok = dpad % 4 == 0 && (DREG > 0 || (d * dv) % 4 == 0);
  const bool vec_k = smem_ok && stage_vec_ok<T>(k + (size_t)t0 * a.ld + head * d, a.ld, d);
  const bool vec_q = smem_ok && stage_vec_ok<T>(q + (size_t)t0 * a.ld + head * d, a.ld, d);
  const bool vec_v = smem_ok && stage_vec_ok<T>(v + (size_t)t0 * a.ld + head * dv, a.ld, dv);
  const bool vec_g = smem_ok && stage_vec_ok<T>(g + (size_t)t0 * a.ld + head * dv, a.ld, dv);
  for (int tb = t0; tb < t1; tb += batch) {
    const int nb = min(batch, t1 - tb);
    __syncthreads();                               // the batch before this one has been read
    stage_rows_f32<T>(kb, dpad, k + (size_t)tb * a.ld + head * d, a.ld, nb, d, 1.f, vec_k);
    if (MODE != 1) stage_rows_f32<T>(qb, dpad, q + (size_t)tb * a.ld + head * d, a.ld, nb, d, a.q_scale, vec_q);
    stage_rows_raw<T>(vb, v + (size_t)tb * a.ld + head * dv, a.ld, nb, dv, vec_v);
    if (MODE != 1) stage_rows_raw<T>(gb, g + (size_t)tb * a.ld + head * dv, a.ld, nb, dv, vec_g);
    if (threadIdx.x < nb) {
      const int t = tb + threadIdx.x;
      s_keep[threadIdx.x] = a.cap * tanhf((a.gates[(size_t)t * 2 * a.heads + head] + bi) / a.cap);
      s_take[threadIdx.x] = log_sigmoid(a.cap * tanhf((a.gates[(size_t)t * 2 * a.heads + a.heads + head] + bf) / a.cap));
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int tt = 0; tt < nb; ++tt) {
        const float gi = s_keep[tt], gf = s_take[tt];
        const float m_new = fmaxf(gf + m, gi);
        s_keep[tt] = expf(gf + m - m_new);
        s_take[tt] = expf(gi - m_new);
        s_em[tt] = expf(-m_new);
        m = m_new;
        fsum += gf;
      }
    }
    __syncthreads();
    for (int tt = 0; tt < nb; ++tt) {
      const float keep = s_keep[tt], take = s_take[tt];
      const float* ks = kb + (size_t)tt * dpad;
      const float* qs = qb + (size_t)tt * dpad;
      for (int i = threadIdx.x; i < d; i += blockDim.x) nvec[i] = keep * nvec[i] + take * ks[i];
      if (MODE != 1) __syncthreads();              // every thread reads n below
      float o = 0.f;
      if (j < dv) {
        const float tv = take * to_f32<T>(vb[(size_t)tt * dv + j]);
        float acc = 0.f, nq = 0.f;
        float acc1 = 0.f, acc2 = 0.f, acc3 = 0.f, nq1 = 0.f, nq2 = 0.f, nq3 = 0.f;
        if (DREG > 0) {
#pragma unroll
          for (int i = 0; i < DP; i += 4) {
            const float4 k4 = *reinterpret_cast<const float4*>(ks + i0 + i);
            Sr[i] = fmaf(keep, Sr[i], k4.x * tv);
            Sr[i + 1] = fmaf(keep, Sr[i + 1], k4.y * tv);
            Sr[i + 2] = fmaf(keep, Sr[i + 2], k4.z * tv);
            Sr[i + 3] = fmaf(keep, Sr[i + 3], k4.w * tv);
            if (MODE != 1) {
              const float4 q4 = *reinterpret_cast<const float4*>(qs + i0 + i);
              const float4 n4 = *reinterpret_cast<const float4*>(nvec + i0 + i);
              acc = fmaf(Sr[i], q4.x, acc);          // four sums side by side: a chain of dependent adds is what
              acc1 = fmaf(Sr[i + 1], q4.y, acc1);    // the walk would otherwise wait for
              acc2 = fmaf(Sr[i + 2], q4.z, acc2);
              acc3 = fmaf(Sr[i + 3], q4.w, acc3);
              nq = fmaf(n4.x, q4.x, nq);
              nq1 = fmaf(n4.y, q4.y, nq1);
              nq2 = fmaf(n4.z, q4.z, nq2);
              nq3 = fmaf(n4.w, q4.w, nq3);
            }
          }
          acc = (acc + acc1) + (acc2 + acc3);
          nq = (nq + nq1) + (nq2 + nq3);
          if (SPLIT == 2 && MODE != 1) {           // the column's other half
            acc += __shfl_xor_sync(0xffffffffu, acc, 16);
            nq += __shfl_xor_sync(0xffffffffu, nq, 16);
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
        o = acc / (fmaxf(fabsf(nq), s_em[tt]) + 1e-6f);
      }
      if (MODE == 1) continue;                     // n[i] is its own thread's, the staged rows are only read
      const float ss = block_sum(i0 == 0 ? o * o : 0.f, red);   // its barriers also put this token's reads of n before the next update
      if (j < dv && i0 == 0) {
        const float gate = to_f32<T>(gb[(size_t)tt * dv + j]);
        const float y = o * rsqrtf(ss / (float)dv + a.eps) * nw / (1.f + expf(-gate));
        ((T*)a.out)[(size_t)(tb + tt) * a.heads * dv + head * dv + j] = from_f32<T>(y);
      }
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
        if (i0 + i < d) dst_S[(size_t)(i0 + i) * dv + j] = Sr[i];
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
// (S, n).  The chain of maxima is scalar: thread 0 follows it once per tile of chunks and leaves every chunk's two
// factors in shared memory; the elements then take eight chunks' loads at a time.
constexpr int kChainTile = 64;

__global__ void mlstm_chain_kernel(MlstmArgs a) {
  __shared__ float s_keep[kChainTile], s_take[kChainTile];
  __shared__ float s_m;
  pdl_wait_block();
  pdl_launch_dependents();
  const int head = blockIdx.x, b = blockIdx.y, d = a.d, dv = a.dv;
  const int e = blockIdx.z * blockDim.x + threadIdx.x;
  const int elems = d * dv + d;
  const int slot = a.seq_slot[b];
  if (slot < 0 || slot >= a.n_slots) return;
  const bool live = e < elems;
  const int q_len = a.seq_qstart[b + 1] - a.seq_qstart[b];
  const int n_chunks = (q_len + a.chunk - 1) / a.chunk;
  const size_t unit = mlstm_unit(d, dv);
  float* cs = a.scratch + ((size_t)b * a.max_chunks * a.heads + head) * unit;   // chunk c: cs + c * per
  const size_t per = (size_t)a.heads * unit;
  float cur = 0.f;
  if (live) cur = e < d * dv ? a.S[((size_t)slot * a.heads + head) * d * dv + e] : a.n[((size_t)slot * a.heads + head) * d + (e - d * dv)];
  if (threadIdx.x == 0) s_m = a.m[(size_t)slot * a.heads + head];
  for (int c0 = 0; c0 < n_chunks; c0 += kChainTile) {
    const int nc = min(kChainTile, n_chunks - c0);
    __syncthreads();
    if (threadIdx.x == 0) {
      float m = s_m;
      for (int i = 0; i < nc; ++i) {
        float* u = cs + (size_t)(c0 + i) * per;
        const bool has = c0 + i + 1 < n_chunks;
        const float M = has ? u[unit - 3] : 0.f, F = has ? u[unit - 2] : 0.f;
        if (e == 0) u[unit - 1] = m;               // the maximum at this chunk's start (block z = 0 writes it)
        const float m_new = has ? fmaxf(F + m, M) : m;
        s_keep[i] = has ? expf(F + m - m_new) : 1.f;
        s_take[i] = has ? expf(M - m_new) : 0.f;
        m = m_new;
      }
      s_m = m;
    }
    __syncthreads();
    if (!live) continue;
    for (int i0 = 0; i0 < nc; i0 += 8) {
      float loc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) loc[i] = (i0 + i < nc && c0 + i0 + i + 1 < n_chunks) ? cs[(size_t)(c0 + i0 + i) * per + e] : 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (i0 + i < nc) {
          cs[(size_t)(c0 + i0 + i) * per + e] = cur;
          cur = s_keep[i0 + i] * cur + s_take[i0 + i] * loc[i];
        }
      }
    }
  }
}

template <typename T, int DREG, int SPLIT>
static int mlstm_run(const MlstmArgs& a, int max_q, cudaStream_t stream) {
  const int d = a.d, dv = a.dv;
  int batch = kMlstmBatch;                       // as many tokens staged at a time as shared memory takes
  while (batch > 1 && mlstm_smem_bytes<T>(d, dv, DREG * SPLIT, batch) > 200 * 1024) batch /= 2;
  const size_t smem = mlstm_smem_bytes<T>(d, dv, DREG * SPLIT, batch);
  if (smem > 200 * 1024) return PE_ERR_UNSUPPORTED_SIZE;
  const int widest = dv > d ? dv : d;
  int threads = (SPLIT * widest + 31) / 32 * 32;
  const int cap_threads = DREG == 64 ? 512 : 1024;
  if (threads > cap_threads) threads = cap_threads;
  if (DREG > 0 && SPLIT * dv > threads) return PE_ERR_UNSUPPORTED_SIZE;
  auto k0 = mlstm_kernel<T, 0, DREG, SPLIT>;
  auto k1 = mlstm_kernel<T, 1, DREG, SPLIT>;
  auto k3 = mlstm_kernel<T, 3, DREG, SPLIT>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(k0, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k3, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  if (a.chunk > 0) {
    const dim3 grid(a.heads, a.n_seqs, a.max_chunks);
    launch(k1, grid, dim3(threads), smem, stream, a, batch);
    const int elems = d * dv + d;
    launch(mlstm_chain_kernel, dim3(a.heads, a.n_seqs, (elems + 255) / 256), dim3(256), 0, stream, a);
    launch(k3, grid, dim3(threads), smem, stream, a, batch);
  } else {
    launch(k0, dim3(a.heads, a.n_seqs, 1), dim3(threads), smem, stream, a, batch);
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
  // 128: two threads a column with 64 rows each (the value size then fills whole half-warps)
  const int reg = (d <= 32) ? 32 : (d <= 64 && dv <= 512 ? 64 : (d <= 128 && dv <= 256 && dv % 16 == 0 ? 128 : 0));
  if (reg == 0 && ((size_t)d * dv + 3 * (size_t)d) * sizeof(float) + 2 * (size_t)dv * 4 > 200 * 1024) return PE_ERR_UNSUPPORTED_SIZE;
  int rc;
#define PE_MLSTM(T)                                                          \
  (reg == 32 ? pe::mlstm_run<T, 32, 1>(a, max_q, stream)                     \
   : reg == 64 ? pe::mlstm_run<T, 64, 1>(a, max_q, stream)                   \
   : reg == 128 ? pe::mlstm_run<T, 64, 2>(a, max_q, stream) : pe::mlstm_run<T, 0, 1>(a, max_q, stream))
  rc = dtype == PE_F32 ? PE_MLSTM(float) : PE_MLSTM(__nv_bfloat16);
#undef PE_MLSTM
  if (rc != PE_OK) return rc;
  PE_LAUNCH_CHECK();
  return PE_OK;
}
