// A linear-recurrence mixer with a matrix state per head (RWKV-style "wkv" time mixing with a data-dependent
// decay), for prompts and for single tokens alike.
//
//   shifted mixes   m_s[t] = h[t] + (h[t-1] - h[t]) * mu_s          h[-1] of a sequence: the state's `prev` row
//   decay           w[t]   = exp(-exp(wlin[t] + w0))                 float32, per head and key channel
//   read            o[t]   = (S + diag(u) k[t] v[t]^T)^T r[t]        the bonus u acts on the current token only
//   update          S     <- diag(w[t]) S + k[t] v[t]^T              float32 state [d_key, d_value] per head
//   out[t]          = o[t] / rms(o[t]) * gnorm * silu(g[t])          per head, eps inside the root
//
// A block owns one head's state in registers and walks the sequence's tokens of this step in order (the read is
// written as o_j = sum_i r_i S_ij + v_j sum_i r_i u_i k_i, the bonus term taken out of the sum over i).  The recurrence, the decay and the head norm are
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

// The same for bfloat16 rows whose width is a multiple of 8 and that start on 16-byte boundaries: eight channels a
// thread, 16-byte loads and stores.
__global__ void token_shift_mix_vec8_kernel(const __nv_bfloat16* x, const float* __restrict__ mu, int n_mix,
                                            const float* prev_state, const int* token_seq, const int* seq_slot,
                                            const int* seq_qstart, __nv_bfloat16* __restrict__ out, int n_tokens, int width,
                                            int n_slots, int* status) {
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
  const __nv_bfloat16* cur = x + (size_t)t * width;
  for (int c = threadIdx.x * 8; c < width; c += blockDim.x * 8) {
    float h[8], dl[8];
    {
      const uint4 raw = *reinterpret_cast<const uint4*>(cur + c);
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h2[e]);
        h[2 * e] = f.x;
        h[2 * e + 1] = f.y;
      }
    }
    if (first) {
      const float4 p0 = *reinterpret_cast<const float4*>(prev_state + (size_t)slot * width + c);
      const float4 p1 = *reinterpret_cast<const float4*>(prev_state + (size_t)slot * width + c + 4);
      const float pp[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
      for (int e = 0; e < 8; ++e) dl[e] = pp[e] - h[e];
    } else {
      const uint4 raw = *reinterpret_cast<const uint4*>(cur + c - width);
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h2[e]);
        dl[2 * e] = f.x - h[2 * e];
        dl[2 * e + 1] = f.y - h[2 * e + 1];
      }
    }
    for (int s = 0; s < n_mix; ++s) {
      const float4 m0 = *reinterpret_cast<const float4*>(mu + (size_t)s * width + c);
      const float4 m1 = *reinterpret_cast<const float4*>(mu + (size_t)s * width + c + 4);
      const float mm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
      uint4 o;
      __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e)
        o2[e] = __floats2bfloat162_rn(fmaf(dl[2 * e], mm[2 * e], h[2 * e]), fmaf(dl[2 * e + 1], mm[2 * e + 1], h[2 * e + 1]));
      *reinterpret_cast<uint4*>(out + ((size_t)s * n_tokens + t) * width + c) = o;
    }
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
//
// A block holds one head's state in registers, a tile of 4 columns x RI rows per thread (the DMAX / 4 column blocks
// times NIB row blocks are the block's threads).  It walks its tokens in batches of TB.  The first DMAX threads are
// also the stagers, one channel each: a stager holds the next batch's raw r, k, v, g and decay input in registers
// (their loads are issued before the current batch's arithmetic, so memory latency hides behind it), and at a batch's
// start turns them into what the arithmetic reads from shared memory: r, k, the decay itself (exponentials taken
// here), r*u*k for the bonus term, v, and silu(g) times the norm's weight.  Then every thread runs the batch's tokens
// through its tile: three multiply-adds per state element and token, with r, k, w of its row block read as 16-byte
// pieces that serve four columns each (a thread that owned a whole column read twelve bytes of shared memory per
// state element and was bound by that); the partial outputs of the row blocks, and their parts of the bonus sum
// sum_i r_i u_i k_i (the same number for every column), are added up by shuffles and the outputs left in shared
// memory; the per-head norm, the gate and the store are then done a token per warp.  Row blocks lie 4 floats apart
// from a multiple of 32 in shared memory, so that the four (or eight) pieces a warp reads at once fall into different
// banks.
template <int DMAX> struct WkvTile {
  static constexpr int NIB = DMAX <= 128 ? 4 : 8;     // row blocks
  static constexpr int RI = DMAX / NIB;               // rows per thread
  static constexpr int NJB = DMAX / 4;                // column blocks
  static constexpr int NT = NJB * NIB;                // threads per block
  static constexpr int TB = 4;                        // tokens per batch
  static constexpr int RS = RI + 4;                   // floats from one row block to the next in shared memory
  static constexpr int ROWW = NIB * RS;
  static constexpr int MIN_BLOCKS = DMAX <= 32 ? 16 : (DMAX == 64 ? 8 : (DMAX == 128 ? 2 : 1));
};

template <typename T> __device__ __forceinline__ float silu_of(float g) { return g / (1.f + expf(-g)); }
// a gate that is rounded to bfloat16 afterwards may take the hardware's approximate exponential and reciprocal
template <> __device__ __forceinline__ float silu_of<__nv_bfloat16>(float g) { return __fdividef(g, 1.0f + __expf(-g)); }

template <typename T, int DMAX, int MODE>
__global__ void __launch_bounds__(WkvTile<DMAX>::NT, MODE == 0 ? 1 : WkvTile<DMAX>::MIN_BLOCKS) wkv_scan_kernel(WkvArgs a) {
  typedef WkvTile<DMAX> TL;
  constexpr int NIB = TL::NIB, RI = TL::RI, NT = TL::NT, TB = TL::TB, RS = TL::RS, NW = NT / 32;
  __shared__ __align__(16) float sr[TB][TL::ROWW], sk[TB][TL::ROWW], sw[TB][TL::ROWW], sb[TB][TL::ROWW];
  __shared__ __align__(16) float sv[TB][DMAX], so[TB][DMAX];
  __shared__ float sg[TB][DMAX];                      // silu(g) times the norm's weight
  const int tid = threadIdx.x, d = a.d;
  const int warp = tid >> 5, lane = tid & 31;
  const int ib = tid % NIB, jb = tid / NIB;          // this thread's row block and column block
  const int head = blockIdx.x, b = blockIdx.y, c = blockIdx.z;
  const int hd = a.heads * d;
  const bool stager = tid < DMAX;                    // as a stager, thread `tid` brings channel `tid` of the head
  const bool live = tid < d;
  const int col = head * d + tid;
  const int spos = (tid / RI) * RS + (tid % RI);     // where channel `tid` lies in a row of sr, sk, sw, sb
  float w0 = 0.f, uj = 0.f, gn = 0.f;
  if (live) {
    w0 = a.w0[col];
    uj = a.u[col];
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
    if (tid == 0) report(a.status, kStatusSlotOutOfRange, b, slot, a.n_slots);
    return;
  }
  const T* R = (const T*)a.r; const T* K = (const T*)a.k; const T* V = (const T*)a.v; const T* G = (const T*)a.g;
  float pr[TB], pk[TB], pv[TB], pg[TB], pw[TB];      // a stager's raw inputs of the batch to come
  auto fetch = [&](int tb) {
#pragma unroll
    for (int e = 0; e < TB; ++e) {
      pr[e] = pk[e] = pv[e] = pg[e] = pw[e] = 0.f;
      if (live && tb + e < t1) {
        const size_t at = (size_t)(tb + e) * a.ld + col;
        pr[e] = to_f32<T>(R[at]);
        pk[e] = to_f32<T>(K[at]);
        pv[e] = to_f32<T>(V[at]);
        if (MODE != 1) pg[e] = to_f32<T>(G[at]);
        pw[e] = a.wlin[(size_t)(tb + e) * hd + col];
      }
    }
  };
  fetch(t0);
  float* slot_state = a.state + ((size_t)slot * a.heads + head) * d * d;
  float* cs = (MODE != 0) ? a.chunk_state + (((size_t)b * a.max_chunks + c) * a.heads + head) * d * d : nullptr;
  const float* start = (MODE == 0) ? slot_state : cs;
  const int row0 = ib * RI, col0 = 4 * jb;
  const bool vec_state = (d % 4 == 0);
  float S[4][RI];                         // S[cc][r]: state element (row0 + r, col0 + cc)
#pragma unroll
  for (int r = 0; r < RI; ++r) {
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
    if (MODE != 1 && row0 + r < d) {
      const float* p = start + (size_t)(row0 + r) * d + col0;
      if (vec_state) {
        if (col0 < d) x = *reinterpret_cast<const float4*>(p);
      } else {
        if (col0 < d) x.x = p[0];
        if (col0 + 1 < d) x.y = p[1];
        if (col0 + 2 < d) x.z = p[2];
        if (col0 + 3 < d) x.w = p[3];
      }
    }
    S[0][r] = x.x; S[1][r] = x.y; S[2][r] = x.z; S[3][r] = x.w;
  }
  float decay_prod = 1.f;   // MODE 1: stager `tid` keeps the product of its channel's decays
  for (int tb = t0; tb < t1; tb += TB) {
    const int nt = min(TB, t1 - tb);
    __syncthreads();                       // the batch before this one has been read to its end
    if (stager) {
#pragma unroll
      for (int e = 0; e < TB; ++e) {
        const float w = (live && e < nt) ? expf(-expf(pw[e] + w0)) : 0.f;
        sr[e][spos] = pr[e];                // channels beyond d hold zeros: their rows of the state stay zero
        sk[e][spos] = pk[e];
        sw[e][spos] = w;
        sv[e][tid] = pv[e];
        if (MODE == 1) {
          if (live && e < nt) decay_prod *= w;
        } else {
          sb[e][spos] = pr[e] * uj * pk[e];
          sg[e][tid] = silu_of<T>(pg[e]) * gn;
        }
      }
    }
    __syncthreads();
    if (stager) fetch(tb + TB);            // on its way while this batch is worked on
    asm volatile("" ::: "memory");         // the compiler may not sink these loads below the arithmetic, to where they are used
#pragma unroll 1
    for (int tt = 0; tt < nt; ++tt) {
      const float4 v4 = *reinterpret_cast<const float4*>(&sv[tt][col0]);
      const float vv[4] = {v4.x, v4.y, v4.z, v4.w};
      const float4* r4 = reinterpret_cast<const float4*>(&sr[tt][ib * RS]);
      const float4* k4 = reinterpret_cast<const float4*>(&sk[tt][ib * RS]);
      const float4* w4 = reinterpret_cast<const float4*>(&sw[tt][ib * RS]);
      const float4* b4 = reinterpret_cast<const float4*>(&sb[tt][ib * RS]);
      float o[4] = {0.f, 0.f, 0.f, 0.f};
      float bonus = 0.f;
#pragma unroll
      for (int q = 0; q < RI / 4; ++q) {
        if (row0 + 4 * q < d) {
          const float4 kq = k4[q], wq = w4[q];
          const float kk[4] = {kq.x, kq.y, kq.z, kq.w}, ww[4] = {wq.x, wq.y, wq.z, wq.w};
          float rr[4] = {0.f, 0.f, 0.f, 0.f};
          if (MODE != 1) {
            const float4 rq = r4[q], bq = b4[q];
            rr[0] = rq.x; rr[1] = rq.y; rr[2] = rq.z; rr[3] = rq.w;
            bonus += (bq.x + bq.y) + (bq.z + bq.w);
          }
#pragma unroll
          for (int e = 0; e < 4; ++e)
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
              if (MODE != 1) o[cc] = fmaf(rr[e], S[cc][4 * q + e], o[cc]);
              S[cc][4 * q + e] = fmaf(ww[e], S[cc][4 * q + e], kk[e] * vv[cc]);
            }
        }
      }
      if (MODE == 1) continue;
#pragma unroll
      for (int m = 1; m < NIB; m <<= 1) {
        bonus += __shfl_xor_sync(0xffffffffu, bonus, m);
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) o[cc] += __shfl_xor_sync(0xffffffffu, o[cc], m);
      }
      if (ib == 0)
        *reinterpret_cast<float4*>(&so[tt][col0]) = make_float4(fmaf(bonus, vv[0], o[0]), fmaf(bonus, vv[1], o[1]),
                                                                fmaf(bonus, vv[2], o[2]), fmaf(bonus, vv[3], o[3]));
    }
    if (MODE == 1) continue;
    __syncthreads();
    // a token per warp: the head's outputs divided by their root mean square, times the norm's weight and the gate
    for (int tt = warp; tt < nt; tt += NW) {
      float ss = 0.f;
      for (int i = lane; i < d; i += 32) ss += so[tt][i] * so[tt][i];
      const float inv = rsqrtf(warp_sum(ss) / (float)d + a.eps);
      const size_t t = (size_t)(tb + tt);
      for (int i = lane; i < d; i += 32) ((T*)a.out)[t * hd + head * d + i] = from_f32<T>(so[tt][i] * inv * sg[tt][i]);
    }
  }
  const bool store_state = MODE == 1 || t1 == q1;   // MODE 0/3: the sequence's last token of this step is here
  if (store_state) {
    float* dst = MODE == 1 ? cs : slot_state;
#pragma unroll
    for (int r = 0; r < RI; ++r) {
      if (row0 + r < d && col0 < d) {
        float* p = dst + (size_t)(row0 + r) * d + col0;
        if (vec_state) {
          *reinterpret_cast<float4*>(p) = make_float4(S[0][r], S[1][r], S[2][r], S[3][r]);
        } else {
          p[0] = S[0][r];
          if (col0 + 1 < d) p[1] = S[1][r];
          if (col0 + 2 < d) p[2] = S[2][r];
          if (col0 + 3 < d) p[3] = S[3][r];
        }
      }
    }
  }
  if (MODE == 1) {
    if (live) a.chunk_decay[(((size_t)b * a.max_chunks + c) * a.heads + head) * d + tid] = decay_prod;
    return;
  }
  if (t1 == q1) {
    // the sequence's last input row becomes `prev`; each head's block copies its share of the width (one block
    // copying all of it, 64 threads wide, was the longest thing a decode step's launch of this kernel did)
    const T* last = (const T*)a.x + (size_t)(q1 - 1) * a.width;
    const int per = (a.width + a.heads - 1) / a.heads;
    const int hi = min(a.width, (head + 1) * per);
    for (int cidx = head * per + tid; cidx < hi; cidx += blockDim.x) a.prev_state[(size_t)slot * a.width + cidx] = to_f32<T>(last[cidx]);
  }
}

// Chain the chunks: on entry chunk_state[c] holds chunk c's end state from zero (every chunk but the sequence's
// last one); on exit it holds chunk c's true start state, chunk 0's being the slot's state.  One thread per state
// element (256 elements a block), chunks in order.
__global__ void wkv_chain_kernel(WkvArgs a) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int head = blockIdx.x, b = blockIdx.y, d = a.d;
  const int e = blockIdx.z * blockDim.x + threadIdx.x;     // this thread's state element
  if (e >= d * d) return;
  const int q_len = a.seq_qstart[b + 1] - a.seq_qstart[b];
  const int n_chunks = (q_len + a.chunk - 1) / a.chunk;
  const int slot = a.seq_slot[b];
  if (slot < 0 || slot >= a.n_slots) return;
  const int i = e / d;
  const size_t per = (size_t)a.heads * d * d, per_decay = (size_t)a.heads * d;
  float* cs = a.chunk_state + ((size_t)b * a.max_chunks * a.heads + head) * d * d + e;       // chunk c: cs[c * per]
  const float* cd = a.chunk_decay + ((size_t)b * a.max_chunks * a.heads + head) * d + i;      // chunk c: cd[c * per_decay]
  float s = a.state[((size_t)slot * a.heads + head) * d * d + e];
  // four chunks' loads in flight at a time; the last chunk of the sequence has left neither end state nor decays
  for (int c0 = 0; c0 < n_chunks; c0 += 4) {
    float local[4], p[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int c = c0 + k;
      const bool has = c + 1 < n_chunks;
      local[k] = has ? cs[(size_t)c * per] : 0.f;
      p[k] = has ? cd[(size_t)c * per_decay] : 0.f;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int c = c0 + k;
      if (c < n_chunks) {
        cs[(size_t)c * per] = s;          // chunk c's true start
        s = fmaf(p[k], s, local[k]);
      }
    }
  }
}

template <typename T, int DMAX>
static int launch_wkv(const WkvArgs& a, int max_q, cudaStream_t stream) {
  if (a.chunk > 0) {
    dim3 grid(a.heads, a.n_seqs, a.max_chunks);
    pe::launch(wkv_scan_kernel<T, DMAX, 1>, grid, WkvTile<DMAX>::NT, 0, stream, a);
    PE_LAUNCH_CHECK();
    pe::launch(wkv_chain_kernel, dim3(a.heads, a.n_seqs, (a.d * a.d + 255) / 256), 256, 0, stream, a);
    PE_LAUNCH_CHECK();
    pe::launch(wkv_scan_kernel<T, DMAX, 3>, grid, WkvTile<DMAX>::NT, 0, stream, a);
    PE_LAUNCH_CHECK();
    return PE_OK;
  }
  pe::launch(wkv_scan_kernel<T, DMAX, 0>, dim3(a.heads, a.n_seqs, 1), WkvTile<DMAX>::NT, 0, stream, a);
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
  const bool vec8 = dtype == PE_BF16 && width % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)out % 16 == 0 &&
                    (uintptr_t)mu % 16 == 0 && (uintptr_t)prev_state % 16 == 0 && ((size_t)n_tokens * width) % 8 == 0;
  if (vec8) {
    pe::launch(pe::token_shift_mix_vec8_kernel, n_tokens, width >= 2048 ? 256 : 128, 0, stream, (const __nv_bfloat16*)x, mu, n_mix,
               prev_state, token_seq, seq_slot, seq_qstart, (__nv_bfloat16*)out, n_tokens, width, n_slots, status);
    PE_LAUNCH_CHECK();
    return PE_OK;
  }
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
