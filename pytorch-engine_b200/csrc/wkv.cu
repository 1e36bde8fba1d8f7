// A linear-recurrence mixer with a matrix state per head (RWKV-style "wkv" time mixing with a data-dependent
// decay), for prompts and for single tokens alike.
//
//   shifted mixes   m_s[t] = h[t] + (h[t-1] - h[t]) * mu_s          h[-1] of a sequence: the state's `prev` row
//   decay           w[t]   = exp(-exp(wlin[t] + w0))                 float32, per head and key channel
//   read            o[t]   = (S + diag(u) k[t] v[t]^T)^T r[t]        the bonus u acts on the current token only
//   update          S     <- diag(w[t]) S + k[t] v[t]^T              float32 state [d_key, d_value] per head
//   out[t]          = o[t] / rms(o[t]) * gnorm * silu(g[t])          per head, eps inside the root
//
// The state's columns (value channels) never mix: thread j of a block owns column j of its head's state in
// registers and walks the sequence's tokens of this step in order.  The recurrence, the decay and the head norm are
// float32 whatever the run dtype; r, k, v, g come from matrix products in the run dtype.  Long prompts are cut into
// chunks that run side by side: the update is linear in S, so a chunk first folds its tokens into a state that
// starts at zero together with the product of its decays, a second kernel chains the chunks' starts
// (S_start[c+1] = diag(P_c) S_start[c] + S_local[c]), and the chunks then produce their outputs from their true
// starts.  Which chunk a token falls into depends on the sequence's own tokens of this step only.
#include "api.h"
#include "common.cuh"

namespace pe {

// ---- token shift ---------------------------------------------------------------------------------------------
// out[s][t][c] = x[t][c] + (x'[t][c] - x[t][c]) * mu[s][c];  grid: tokens, block: threads over the width.
template <typename T>
__global__ void token_shift_mix_kernel(const T* x, const float* __restrict__ mu, int n_mix, const float* prev_state,
                                       const int* token_seq, const int* seq_slot, const int* seq_qstart,
                                       T* __restrict__ out, int n_tokens, int width, int n_slots, int* status) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  if (t >= n_tokens) return;
  const int b = token_seq[t];
  const bool first = t == seq_qstart[b];
  const int slot = seq_slot[b];
  if (first && (slot < 0 || slot >= n_slots)) {
    if (threadIdx.x == 0) report(status, kStatusSlotOutOfRange, t, slot, n_slots);
    return;
  }
  const T* cur = x + (size_t)t * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float h = to_f32<T>(cur[c]);
    const float hp = first ? prev_state[(size_t)slot * width + c] : to_f32<T>(cur[c - width]);
    const float dlt = hp - h;
    for (int s = 0; s < n_mix; ++s)
      out[((size_t)s * n_tokens + t) * width + c] = from_f32<T>(fmaf(dlt, mu[(size_t)s * width + c], h));
  }
}

// y = tanh(y) in place (the activation inside the decay's low-rank projection)
template <typename T>
__global__ void tanh_kernel(T* y, size_t n) {
  pdl_wait_block();
  pdl_launch_dependents();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    y[i] = from_f32<T>(tanhf(to_f32<T>(y[i])));
}

// ---- the recurrence ----------------------------------------------------------------------------------------------
struct WkvArgs {
  const void* r; const void* k; const void* v; const void* g;   // [n_tokens, ld] in the run dtype
  long long ld;
  const float* wlin;            // [n_tokens, heads*d] float32: the decay projection before its offset
  const float* w0;              // [heads*d]
  const float* u;               // [heads*d]
  const float* gnorm;           // [heads*d]
  float eps;
  void* out;                    // [n_tokens, heads*d] in the run dtype
  float* state;                 // [slots, heads, d, d]
  float* prev_state;            // [slots, width]
  const void* x; int width;     // the mixer's input rows: the last one of each sequence becomes `prev`
  const int* seq_slot; const int* seq_qstart;
  int n_seqs, heads, d, n_slots;
  int chunk;                    // tokens per chunk (phases 1-3), 0: the whole step in one go
  int max_chunks;
  float* chunk_state;           // [n_seqs, max_chunks, heads, d, d]  local end states, then true start states
  float* chunk_decay;           // [n_seqs, max_chunks, heads, d]     product of the chunk's decays
  int* status;
};

// MODE 0: whole step (start from the slot's state, write outputs, write the state back)
// MODE 1: chunk c from a zero state: leaves its end state and decay product           (no outputs)
// MODE 3: chunk c from its true start (chunk_state, as the chain kernel left it): writes outputs; the last chunk
//         writes the slot's state, which no block of this launch reads
template <typename T, int DMAX, int MODE>
__global__ void __launch_bounds__(DMAX) wkv_scan_kernel(WkvArgs a) {
  __shared__ float sr[2][DMAX], sk[2][DMAX], sw[2][DMAX], su[DMAX], red[32];
  const int j = threadIdx.x, d = a.d;
  const int head = blockIdx.x, b = blockIdx.y, c = blockIdx.z;
  const int hd = a.heads * d;
  const int col = head * d + j;
  const bool live = j < d;
  // constants of the head: on their way before the wait
  float w0 = 0.f, gn = 0.f;
  if (live) {
    w0 = a.w0[col];
    su[j] = a.u[col];
    gn = a.gnorm[col];
  }
  pdl_wait_block();
  pdl_launch_dependents();
  const int q0 = a.seq_qstart[b], q1 = a.seq_qstart[b + 1];
  int t0 = q0, t1 = q1;
  if (MODE != 0) {
    t0 = q0 + c * a.chunk;
    t1 = min(q1, t0 + a.chunk);
    if (t0 >= q1) return;
    if (MODE == 1 && t1 == q1) return;   // nothing follows the sequence's last chunk: its end state from zero is not needed
  }
  const int slot = a.seq_slot[b];
  if (slot < 0 || slot >= a.n_slots) {
    if (j == 0) report(a.status, kStatusSlotOutOfRange, b, slot, a.n_slots);
    return;
  }
  float S[DMAX];
  float* slot_state = a.state + ((size_t)slot * a.heads + head) * d * d;
  float* cs = (MODE != 0) ? a.chunk_state + (((size_t)b * a.max_chunks + c) * a.heads + head) * d * d : nullptr;
  const float* start = (MODE == 0) ? slot_state : cs;
#pragma unroll
  for (int i = 0; i < DMAX; ++i) S[i] = (MODE != 1 && live && i < d) ? start[(size_t)i * d + j] : 0.f;
  float decay_prod = 1.f;   // MODE 1: thread i keeps the product of w[.][i]
  const T* R = (const T*)a.r; const T* K = (const T*)a.k; const T* V = (const T*)a.v; const T* G = (const T*)a.g;
  auto stage = [&](int t, int buf) {
    if (live) {
      const size_t at = (size_t)t * a.ld + col;
      sr[buf][j] = to_f32<T>(R[at]);
      sk[buf][j] = to_f32<T>(K[at]);
      sw[buf][j] = expf(-expf(a.wlin[(size_t)t * hd + col] + w0));
    }
  };
  stage(t0, 0);
  for (int t = t0; t < t1; ++t) {
    const int buf = (t - t0) & 1;
    __syncthreads();                       // this token's r, k, w are staged; the other buffer is free
    if (t + 1 < t1) stage(t + 1, buf ^ 1);
    const float vj = live ? to_f32<T>(V[(size_t)t * a.ld + col]) : 0.f;
    if (MODE == 1) {
      if (live) decay_prod *= sw[buf][j];
#pragma unroll
      for (int i = 0; i < DMAX; ++i)
        if (i < d) S[i] = fmaf(sw[buf][i], S[i], sk[buf][i] * vj);
      continue;
    }
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < DMAX; ++i) {
      if (i < d) {
        const float kv = sk[buf][i] * vj;
        o = fmaf(sr[buf][i], fmaf(su[i], kv, S[i]), o);
        S[i] = fmaf(sw[buf][i], S[i], kv);
      }
    }
    // the head's outputs divided by their root mean square, times the norm's weight and the gate
    const float ss = block_sum(live ? o * o : 0.f, red);
    if (live) {
      const float inv = rsqrtf(ss / (float)d + a.eps);
      const float gl = to_f32<T>(G[(size_t)t * a.ld + col]);
      const float gate = gl / (1.f + expf(-gl));
      ((T*)a.out)[(size_t)t * hd + col] = from_f32<T>(o * inv * gn * gate);
    }
  }
  if (MODE == 1) {
    if (live) {
#pragma unroll
      for (int i = 0; i < DMAX; ++i)
        if (i < d) cs[(size_t)i * d + j] = S[i];
      a.chunk_decay[(((size_t)b * a.max_chunks + c) * a.heads + head) * d + j] = decay_prod;
    }
    return;
  }
  if (t1 == q1) {   // the sequence's last token of this step is here: the state goes back to the slot
    if (live) {
#pragma unroll
      for (int i = 0; i < DMAX; ++i)
        if (i < d) slot_state[(size_t)i * d + j] = S[i];
    }
    if (head == 0) {
      const T* last = (const T*)a.x + (size_t)(q1 - 1) * a.width;
      for (int cidx = j; cidx < a.width; cidx += blockDim.x) a.prev_state[(size_t)slot * a.width + cidx] = to_f32<T>(last[cidx]);
    }
  }
}

// Chain the chunks: on entry chunk_state[c] holds chunk c's end state from zero (every chunk but the sequence's
// last one); on exit it holds chunk c's true start state, chunk 0's being the slot's state.  One thread per state
// element, chunks in order.
__global__ void wkv_chain_kernel(WkvArgs a) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int head = blockIdx.x, b = blockIdx.y, d = a.d;
  const int q_len = a.seq_qstart[b + 1] - a.seq_qstart[b];
  const int n_chunks = (q_len + a.chunk - 1) / a.chunk;
  const int slot = a.seq_slot[b];
  if (slot < 0 || slot >= a.n_slots) return;
  const float* slot_state = a.state + ((size_t)slot * a.heads + head) * d * d;
  for (int e = threadIdx.x; e < d * d; e += blockDim.x) {
    const int i = e / d;
    float s = slot_state[e];
    for (int c = 0; c < n_chunks; ++c) {
      const size_t at = ((size_t)b * a.max_chunks + c) * a.heads + head;
      float local = 0.f, p = 0.f;
      if (c + 1 < n_chunks) {
        local = a.chunk_state[at * d * d + e];
        p = a.chunk_decay[at * d + i];
      }
      a.chunk_state[at * d * d + e] = s;   // chunk c's true start
      s = fmaf(p, s, local);
    }
  }
}

template <typename T, int DMAX>
static int launch_wkv(const WkvArgs& a, int max_q, cudaStream_t stream) {
  if (a.chunk > 0) {
    dim3 grid(a.heads, a.n_seqs, a.max_chunks);
    pe::launch(wkv_scan_kernel<T, DMAX, 1>, grid, DMAX, 0, stream, a);
    PE_LAUNCH_CHECK();
    pe::launch(wkv_chain_kernel, dim3(a.heads, a.n_seqs), 256, 0, stream, a);
    PE_LAUNCH_CHECK();
    pe::launch(wkv_scan_kernel<T, DMAX, 3>, grid, DMAX, 0, stream, a);
    PE_LAUNCH_CHECK();
    return PE_OK;
  }
  pe::launch(wkv_scan_kernel<T, DMAX, 0>, dim3(a.heads, a.n_seqs, 1), DMAX, 0, stream, a);
  PE_LAUNCH_CHECK();
  return PE_OK;
}

template <typename T>
static int dispatch_wkv(const WkvArgs& a, int max_q, cudaStream_t stream) {
  if (a.d <= 32) return launch_wkv<T, 32>(a, max_q, stream);
  if (a.d <= 64) return launch_wkv<T, 64>(a, max_q, stream);
  if (a.d <= 128) return launch_wkv<T, 128>(a, max_q, stream);
  if (a.d <= 256) return launch_wkv<T, 256>(a, max_q, stream);
  return PE_ERR_UNSUPPORTED_SIZE;
}

}  // namespace pe

extern "C" int pe_token_shift_mix(int dtype, const void* x, const float* mu, int n_mix, const float* prev_state,
                                  const int* token_seq, const int* seq_slot, const int* seq_qstart, void* out,
                                  int n_tokens, int width, int n_slots, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return PE_OK;
  if (width <= 0 || n_mix <= 0) return PE_ERR_BAD_ARGUMENT;
  const int threads = width >= 1024 ? 256 : 128;
  if (dtype == PE_F32)
    pe::launch(pe::token_shift_mix_kernel<float>, n_tokens, threads, 0, stream, (const float*)x, mu, n_mix, prev_state, token_seq,
               seq_slot, seq_qstart, (float*)out, n_tokens, width, n_slots, status);
  else if (dtype == PE_BF16)
    pe::launch(pe::token_shift_mix_kernel<__nv_bfloat16>, n_tokens, threads, 0, stream, (const __nv_bfloat16*)x, mu, n_mix,
               prev_state, token_seq, seq_slot, seq_qstart, (__nv_bfloat16*)out, n_tokens, width, n_slots, status);
  else
    return PE_ERR_UNSUPPORTED_DTYPE;
  PE_LAUNCH_CHECK();
  return PE_OK;
}

extern "C" int pe_tanh_inplace(int dtype, void* y, long long n, cudaStream_t stream) {
  if (n <= 0) return PE_OK;
  const int threads = 256;
  long long blocks = (n + threads - 1) / threads;
  if (blocks > pe::kSMs * 16) blocks = pe::kSMs * 16;
  if (dtype == PE_F32) pe::launch(pe::tanh_kernel<float>, (int)blocks, threads, 0, stream, (float*)y, (size_t)n);
  else if (dtype == PE_BF16) pe::launch(pe::tanh_kernel<__nv_bfloat16>, (int)blocks, threads, 0, stream, (__nv_bfloat16*)y, (size_t)n);
  else return PE_ERR_UNSUPPORTED_DTYPE;
  PE_LAUNCH_CHECK();
  return PE_OK;
}

// Floats of scratch that the chunked form needs for `max_chunks` chunks per sequence.
extern "C" long long pe_wkv_scratch_floats(int n_seqs, int heads, int d, int max_chunks) {
  return (long long)n_seqs * max_chunks * heads * ((long long)d * d + d);
}

// chunk > 0: prompts cut into chunks of that many tokens (scratch from pe_wkv_scratch_floats, max_chunks >=
// ceil(max_q / chunk)); chunk == 0: each sequence's tokens in one go (single tokens, short prompts).
extern "C" int pe_wkv_recurrence(int dtype, const void* r, const void* k, const void* v, const void* g, long long ld,
                                 const float* wlin, const float* w0, const float* u, const float* gnorm, float eps,
                                 void* out, float* state, float* prev_state, const void* x, int width,
                                 const int* seq_slot, const int* seq_qstart, int n_seqs, int max_q, int heads, int d,
                                 int n_slots, int chunk, int max_chunks, float* scratch, int* status,
                                 cudaStream_t stream) {
  if (n_seqs <= 0) return PE_OK;
  if (heads <= 0 || d <= 0 || width <= 0 || n_seqs > 65535) return PE_ERR_BAD_ARGUMENT;
  pe::WkvArgs a;
  a.r = r; a.k = k; a.v = v; a.g = g; a.ld = ld; a.wlin = wlin; a.w0 = w0; a.u = u; a.gnorm = gnorm; a.eps = eps;
  a.out = out; a.state = state; a.prev_state = prev_state; a.x = x; a.width = width;
  a.seq_slot = seq_slot; a.seq_qstart = seq_qstart; a.n_seqs = n_seqs; a.heads = heads; a.d = d; a.n_slots = n_slots;
  a.chunk = 0; a.max_chunks = 1; a.chunk_state = nullptr; a.chunk_decay = nullptr; a.status = status;
  if (chunk > 0) {
    if (!scratch || max_chunks <= 0 || (long long)max_chunks * chunk < max_q || max_chunks > 65535) return PE_ERR_BAD_ARGUMENT;
    a.chunk = chunk; a.max_chunks = max_chunks;
    a.chunk_state = scratch;
    a.chunk_decay = scratch + (size_t)n_seqs * max_chunks * heads * d * d;
  }
  if (dtype == PE_F32) return pe::dispatch_wkv<float>(a, max_q, stream);
  if (dtype == PE_BF16) return pe::dispatch_wkv<__nv_bfloat16>(a, max_q, stream);
  return PE_ERR_UNSUPPORTED_DTYPE;
}
