// A matrix memory per head with exponential gates and a running stabiliser (the mLSTM cell), as a
// recurrence over a state kept per request:
//
//   m_t = max(f_t + m_(t-1), i_t)                       i_t, f_t: logarithms of the input and forget gates
//   a_t = exp(f_t + m_(t-1) - m_t),  b_t = exp(i_t - m_t)
//   S_t = a_t S_(t-1) + b_t k_t v_t^T                   S is [D, DV] per head
//   n_t = a_t n_(t-1) + b_t k_t                         n is [D]
//   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + floor)
//
// with S = 0, n = 0 and m = 0 at the start of a sequence.  n is kept as one more column of S (the
// column of a value that is always 1), so that one thread per column serves both; a request's state
// is [heads, D, DV + 1] floats followed by [heads] stabilisers.
//
// Three kernels.  (1) gates: the gate projections (float32, [tokens, 2 heads]: input gates, then forget
// gates) get their bias, the cap c tanh(z / c) and, the forget gate, the logarithm of the sigmoid; the
// stabiliser is carried along the sequence's tokens (a scan, 128 tokens at a time); a_t, b_t replace the projections and m_t goes to a
// buffer of its own.  (2) recurrence: a CTA takes one sequence, one head and a block of columns; thread j
// keeps column j of the state (D floats) in registers, from the request's slot and back.  It writes the
// numerators S^T q (float32) and, from the extra column, n . q.  (3) output: the division, every head's
// unit-RMS norm, the weight, the sigmoid gate and a constant factor, into the activation type.
//
// Long portions are cut in three passes so that a sequence is not one serial chain (the recurrence is linear
// in the state once a_t and b_t are known): (a) every chunk of C tokens sums its own contribution to the state
// from zero, (b) the chunks' states are chained, S_c = (product of the chunk's a_t) S_(c-1) + dS_c, (c) every
// chunk replays its tokens from its starting state and writes the outputs.  This differs from the serial order
// only in the rounding of the sums.
//
// A sequence's tokens are contiguous and in order in a step; CTAs find them by searching the step's
// token -> sequence map.  Gates, stabiliser, state, sums and norms are float32; q, k and v are read from
// the projection buffer in the activation type.
#include "common.cuh"

#ifndef RL_MM_DIM
#error "compile with -DRL_MM_DIM=<key size>"
#endif

namespace rl {

constexpr int kD = RL_MM_DIM;
static_assert(kD >= 1 && kD <= 256, "key size out of range");
constexpr int kTok = kD > 128 ? 8 : 16;          // tokens staged in shared memory at a time
constexpr int kGateThreads = 128;

// First token index t in [0, n) with seq_of_token[t] >= s.
__device__ __forceinline__ int first_token_of(const int32_t* __restrict__ seq_of_token, int n, int s) {
  int lo = 0, hi = n;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (seq_of_token[mid] < s) lo = mid + 1;
    else hi = mid;
  }
  return lo;
}

// The same for s and s + 1 at once (the two searches' loads in flight together): the sequence's tokens are [b, e).
__device__ __forceinline__ void tokens_of(const int32_t* __restrict__ seq_of_token, int n, int s, int& b, int& e) {
  int lo0 = 0, hi0 = n, lo1 = 0, hi1 = n;
  while (lo0 < hi0 || lo1 < hi1) {
    const int m0 = (lo0 + hi0) >> 1, m1 = (lo1 + hi1) >> 1;
    const int v0 = lo0 < hi0 ? seq_of_token[m0] : 0, v1 = lo1 < hi1 ? seq_of_token[m1] : 0;
    if (lo0 < hi0) {
      if (v0 < s) lo0 = m0 + 1;
      else hi0 = m0;
    }
    if (lo1 < hi1) {
      if (v1 < s + 1) lo1 = m1 + 1;
      else hi1 = m1;
    }
  }
  b = lo0;
  e = lo1;
}

__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float capped(float z, float cap) { return cap > 0.f ? cap * tanhf(z / cap) : z; }

struct MemoryLayout {
  int heads, dv;
  __host__ __device__ size_t plane() const { return static_cast<size_t>(kD) * (dv + 1); }
  __host__ __device__ size_t slot_floats() const { return heads * plane() + heads; }
};

// ---------------------------------------------------------------- (1) gates and stabiliser
// gates [tokens, 2 heads] float32 in place: (z_i, z_f) -> (b_t, a_t); stab [tokens, heads] <- m_t.
__global__ void __launch_bounds__(kGateThreads)
memory_gates_kernel(float* __restrict__ gates, const float* __restrict__ bias_i, const float* __restrict__ bias_f,
                    float cap, const int32_t* __restrict__ seq_of_token, const int32_t* __restrict__ state_slot,
                    float* __restrict__ state, float* __restrict__ stab, int tokens, MemoryLayout lay) {
  pdl_launch();
  pdl_wait();
  __shared__ float wi[kGateThreads / 32], wf[kGateThreads / 32], sm[kGateThreads + 1];
  const int head = blockIdx.x, seq = blockIdx.y;
  const int t_begin = first_token_of(seq_of_token, tokens, seq);
  const int t_end = first_token_of(seq_of_token, tokens, seq + 1);
  if (t_begin >= t_end) return;
  float* m_state = state + static_cast<size_t>(state_slot[seq]) * lay.slot_floats() + lay.heads * lay.plane() + head;
  const float bi = bias_i != nullptr ? bias_i[head] : 0.f, bf = bias_f != nullptr ? bias_f[head] : 0.f;
  if (threadIdx.x == 0) sm[0] = *m_state;
  for (int t0 = t_begin; t0 < t_end; t0 += kGateThreads) {
    const int n = min(kGateThreads, t_end - t0);
    const int t = t0 + threadIdx.x;
    float gi = 0.f, gf = 0.f;
    if (threadIdx.x < n) {
      float* row = gates + static_cast<size_t>(t) * (2 * lay.heads);
      gi = capped(row[head] + bi, cap);
      gf = log_sigmoid(capped(row[lay.heads + head] + bf, cap));
    }
    // The stabiliser along the tokens as a scan: token j maps m to max(f_j + m, i_j); two such maps in a row,
    // (F1, I1) then (F2, I2), are the map (F1 + F2, max(I1 + F2, I2)).  Within a warp by shuffles, then over
    // the warps' totals; sm[j + 1] is m after token j.
    float F = threadIdx.x < n ? gf : 0.f, I = threadIdx.x < n ? gi : -INFINITY;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float Fp = __shfl_up_sync(0xffffffffu, F, o), Ip = __shfl_up_sync(0xffffffffu, I, o);
      if (lane >= o) {
        I = fmaxf(Ip + F, I);
        F = Fp + F;
      }
    }
    if (lane == 31) {
      wf[warp] = F;
      wi[warp] = I;
    }
    __syncthreads();
    float PF = 0.f, PI = -INFINITY;   // the map of all tokens of the warps before this one
    for (int w = 0; w < warp; ++w) {
      PI = fmaxf(PI + wf[w], wi[w]);
      PF += wf[w];
    }
    if (threadIdx.x < n) sm[threadIdx.x + 1] = fmaxf((PF + F) + sm[0], fmaxf(PI + F, I));
    __syncthreads();
    if (threadIdx.x < n) {
      const float m_prev = sm[threadIdx.x], m_new = sm[threadIdx.x + 1];
      float* row = gates + static_cast<size_t>(t) * (2 * lay.heads);
      row[head] = expf(gi - m_new);
      row[lay.heads + head] = expf(gf + m_prev - m_new);
      stab[static_cast<size_t>(t) * lay.heads + head] = m_new;
    }
    __syncthreads();
    if (threadIdx.x == 0) sm[0] = sm[n];
  }
  __syncthreads();
  if (threadIdx.x == 0) *m_state = sm[0];
}

// ---------------------------------------------------------------- (2) the recurrence
template <typename T>
struct MemoryArgs {
  const T* qkv;           // [tokens, ld]: q at q_col + h * D, k at k_col + h * D, v at v_col + h * DV
  int ld, q_col, k_col, v_col;
  float q_scale;
  const float* gates;     // [tokens, 2 heads]: b_t, then a_t
  const int32_t* seq_of_token;
  const int32_t* state_slot;
  float* state;           // [slots] x ([heads, D, DV + 1] + [heads])
  float* num;             // [tokens, heads * DV]: S^T q
  float* qn;              // [tokens, heads]: n . q
  float* chunk_state;     // [sequences, chunks, heads, D, DV + 1] (chunked passes only)
  int tokens, chunk, max_chunks;
  MemoryLayout lay;
};

// mode 0: the whole sequence serially from the slot's state (state written back)
// mode 1: chunk c from zero, no outputs; the chunk's sum goes to chunk_state[seq][c]
// mode 3: chunk c from its starting state as the chain pass left it (chunk_state[seq][c - 1]: the state after
//         chunk c - 1; for c = 0 the slot's state, which the chain pass has copied to the entry of the last
//         chunk, since the last chunk's CTA overwrites the slot), outputs written; the last chunk writes the slot
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
memory_recurrence_kernel(const MemoryArgs<T> a) {
  pdl_launch();
  pdl_wait();
  __shared__ __align__(16) float qs[kTok][kD];
  __shared__ __align__(16) float ks[kTok][kD];       // b_t k_t
  __shared__ float as[kTok];
  __shared__ float vs[kTok][256];      // this thread's value of each staged token (asked for all at once)
  const int seq = blockIdx.z, head = blockIdx.y % a.lay.heads, c = blockIdx.y / a.lay.heads;
  const int dv = a.lay.dv;
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  const bool mine = col <= dv;         // column dv is n
  int seq_begin, seq_end;
  tokens_of(a.seq_of_token, a.tokens, seq, seq_begin, seq_end);
  if (seq_begin >= seq_end) return;
  int t_begin = seq_begin, t_end = seq_end;
  if (MODE != 0) {
    t_begin = seq_begin + c * a.chunk;
    t_end = min(seq_end, t_begin + a.chunk);
    if (t_begin >= seq_end) return;
  }
  const bool last_chunk = t_end == seq_end;
  if (MODE == 1 && last_chunk) return;             // nobody starts from the state after the last chunk
  float* plane = a.state + static_cast<size_t>(a.state_slot[seq]) * a.lay.slot_floats() + head * a.lay.plane();
  float* chunk_plane = a.chunk_state == nullptr ? nullptr
      : a.chunk_state + ((static_cast<size_t>(seq) * a.max_chunks + c) * a.lay.heads + head) * a.lay.plane();
  float S[kD];
  if (MODE == 1) {
#pragma unroll
    for (int i = 0; i < kD; ++i) S[i] = 0.f;
  } else {
    const float* from = plane;
    if (MODE == 3 && c > 0) from = chunk_plane - static_cast<size_t>(a.lay.heads) * a.lay.plane();
    else if (MODE == 3 && !last_chunk) {
      const int chunks = (seq_end - seq_begin + a.chunk - 1) / a.chunk;
      from = chunk_plane + static_cast<size_t>(chunks - 1) * a.lay.heads * a.lay.plane();
    }
#pragma unroll
    for (int i = 0; i < kD; ++i) S[i] = mine ? from[static_cast<size_t>(i) * (dv + 1) + col] : 0.f;
  }

  for (int tb = t_begin; tb < t_end; tb += kTok) {
    const int nt = min(kTok, t_end - tb);
    __syncthreads();
    for (int i = threadIdx.x; i < nt * kD; i += blockDim.x) {
      const int tt = i / kD, d = i - tt * kD;
      const T* row = a.qkv + static_cast<size_t>(tb + tt) * a.ld;
      const float b = a.gates[static_cast<size_t>(tb + tt) * (2 * a.lay.heads) + head];
      if (MODE != 1) qs[tt][d] = to_float(row[a.q_col + head * kD + d]) * a.q_scale;
      ks[tt][d] = to_float(row[a.k_col + head * kD + d]) * b;
    }
    for (int tt = threadIdx.x; tt < nt; tt += blockDim.x)
      as[tt] = a.gates[static_cast<size_t>(tb + tt) * (2 * a.lay.heads) + a.lay.heads + head];
#pragma unroll
    for (int tt = 0; tt < kTok; ++tt) {
      float v = col == dv ? 1.f : 0.f;
      if (tt < nt && col < dv) v = to_float(a.qkv[static_cast<size_t>(tb + tt) * a.ld + a.v_col + head * dv + col]);
      vs[tt][threadIdx.x] = v;
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float v = vs[tt][threadIdx.x];
      const float decay = as[tt];
      float o = 0.f;
      float o1 = 0.f, o2 = 0.f, o3 = 0.f;        // four sums side by side: one chain of kD dependent adds would be the limit
      if (kD % 4 == 0) {
        // keys and queries four at a time: every lane reads the same words, and one 16-byte read serves four
        // updates (read one by one, the shared-memory pipe is the limit, not the arithmetic)
        const float4* k4 = reinterpret_cast<const float4*>(ks[tt]);
        const float4* q4 = reinterpret_cast<const float4*>(qs[tt]);
#pragma unroll
        for (int i = 0; i < kD / 4; ++i) {
          const float4 kk = k4[i];
          S[4 * i] = fmaf(decay, S[4 * i], kk.x * v);
          S[4 * i + 1] = fmaf(decay, S[4 * i + 1], kk.y * v);
          S[4 * i + 2] = fmaf(decay, S[4 * i + 2], kk.z * v);
          S[4 * i + 3] = fmaf(decay, S[4 * i + 3], kk.w * v);
          if (MODE != 1) {
            const float4 qq = q4[i];
            o = fmaf(S[4 * i], qq.x, o);
            o1 = fmaf(S[4 * i + 1], qq.y, o1);
            o2 = fmaf(S[4 * i + 2], qq.z, o2);
            o3 = fmaf(S[4 * i + 3], qq.w, o3);
          }
        }
        o = (o + o1) + (o2 + o3);
      } else {
#pragma unroll
        for (int i = 0; i < kD; ++i) {
          S[i] = fmaf(decay, S[i], ks[tt][i] * v);
          if (MODE != 1) o = fmaf(S[i], qs[tt][i], o);
        }
      }
      if (MODE != 1) {
        if (col < dv) a.num[static_cast<size_t>(tb + tt) * (a.lay.heads * dv) + head * dv + col] = o;
        else if (col == dv) a.qn[static_cast<size_t>(tb + tt) * a.lay.heads + head] = o;
      }
    }
  }
  if (!mine) return;
  float* to = MODE == 1 ? chunk_plane : ((MODE == 0 || last_chunk) ? plane : nullptr);
  if (to != nullptr) {
#pragma unroll
    for (int i = 0; i < kD; ++i) to[static_cast<size_t>(i) * (dv + 1) + col] = S[i];
  }
}

// The chain pass: chunk_state[seq][c] <- (product of chunk c's a_t) * (state after chunk c - 1) + chunk_state[seq][c],
// in order of c.  One thread per element of a head's state; the products of the a_t are formed by repeated
// multiplication in token order, as the recurrence applies them (dynamic shared memory: max_chunks floats).
__global__ void memory_chain_kernel(const float* __restrict__ gates, const int32_t* __restrict__ seq_of_token,
                                    const int32_t* __restrict__ state_slot, const float* __restrict__ state,
                                    float* __restrict__ chunk_state, int tokens, int chunk, int max_chunks,
                                    MemoryLayout lay) {
  pdl_launch();
  pdl_wait();
  const int seq = blockIdx.z, head = blockIdx.y;
  const size_t e = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t plane = lay.plane();
  const int t_begin = first_token_of(seq_of_token, tokens, seq);
  const int t_end = first_token_of(seq_of_token, tokens, seq + 1);
  const int n = t_end - t_begin;
  const int chunks = (n + chunk - 1) / chunk;
  // the chunks' decays side by side, a thread per chunk (every chunk before the last is full)
  extern __shared__ float chunk_decay[];
  for (int c = threadIdx.x; c + 1 < chunks; c += blockDim.x) {
    float decay = 1.f;
    for (int t = t_begin + c * chunk; t < t_begin + (c + 1) * chunk; ++t)
      decay *= gates[static_cast<size_t>(t) * (2 * lay.heads) + lay.heads + head];
    chunk_decay[c] = decay;
  }
  __syncthreads();
  if (e >= plane) return;
  float prev = state[static_cast<size_t>(state_slot[seq]) * lay.slot_floats() + head * plane + e];
  if (chunks >= 2)     // the starting state of chunk 0, kept where no chunk's own sum lies
    chunk_state[((static_cast<size_t>(seq) * max_chunks + chunks - 1) * lay.heads + head) * plane + e] = prev;
  const size_t step = static_cast<size_t>(lay.heads) * plane;          // from a chunk's entry to the next chunk's
  float* p = chunk_state + (static_cast<size_t>(seq) * max_chunks * lay.heads + head) * plane + e;
  constexpr int kAhead = 8;           // the chunks' sums are asked for so many at a time, then chained
  for (int c0 = 0; c0 + 1 < chunks; c0 += kAhead) {
    float own[kAhead];
#pragma unroll
    for (int i = 0; i < kAhead; ++i) own[i] = c0 + i + 1 < chunks ? p[(c0 + i) * step] : 0.f;
#pragma unroll
    for (int i = 0; i < kAhead; ++i) {
      if (c0 + i + 1 < chunks) {
        prev = fmaf(chunk_decay[c0 + i], prev, own[i]);
        p[(c0 + i) * step] = prev;
      }
    }
  }
}

// ---------------------------------------------------------------- (3) division, unit norm, weight, gate
// A warp per (token, head): a CTA takes one token and as many heads as it has warps.
template <typename TA, typename TW>
__global__ void __launch_bounds__(128)
memory_output_kernel(const float* __restrict__ num, const float* __restrict__ qn, const float* __restrict__ stab,
                     const TA* __restrict__ gate, int ld_gate, const TW* __restrict__ w, TA* __restrict__ out,
                     int ld_out, int heads, int dv, float eps, float floor, float out_scale) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int h = blockIdx.y * nwarps + warp; h < heads; h += gridDim.y * nwarps) {
    const float den = fmaxf(fabsf(qn[static_cast<size_t>(t) * heads + h]), expf(-stab[static_cast<size_t>(t) * heads + h])) + floor;
    const float* o = num + static_cast<size_t>(t) * heads * dv + h * dv;
    float q = 0.f;
    for (int d = lane; d < dv; d += 32) {
      const float v = o[d] / den;
      q += v * v;
    }
    const float r = rsqrtf(warp_sum(q) / static_cast<float>(dv) + eps);
    for (int d = lane; d < dv; d += 32) {
      const int c = h * dv + d;
      float y = o[d] / den * r * to_float(w[c]) * out_scale;
      if (gate != nullptr) y *= 1.f / (1.f + expf(-to_float(gate[static_cast<size_t>(t) * ld_gate + c])));
      out[static_cast<size_t>(t) * ld_out + c] = from_float<TA>(y);
    }
  }
}

// chunk_state null or max_chunks <= 1: every sequence is one serial chain.  Otherwise sequences are cut into
// chunks of `chunk` tokens (max_chunks = the most chunks any sequence of the step has) and chunk_state holds
// [sequences, max_chunks, heads, D, DV + 1] floats.
template <typename T>
int launch_recurrence(const MemoryArgs<T>& a, int sequences, cudaStream_t stream) {
  const int cols = a.lay.dv + 1, heads = a.lay.heads;
  // one CTA for all of a head's columns while they fit 256 threads (a head of 128 values has 129 columns)
  const int th = cols <= 256 ? (cols + 31) / 32 * 32 : 128;
  const int col_blocks = (cols + th - 1) / th;
  if (a.chunk_state == nullptr || a.max_chunks <= 1)
    return static_cast<int>(launch_kernel(memory_recurrence_kernel<T, 0>, dim3(col_blocks, heads, sequences), dim3(th), 0,
                                          stream, a));
  cudaError_t e = launch_kernel(memory_recurrence_kernel<T, 1>, dim3(col_blocks, heads * a.max_chunks, sequences),
                                dim3(th), 0, stream, a);
  if (e != cudaSuccess) return static_cast<int>(e);
  const int plane = static_cast<int>(a.lay.plane());
  e = launch_kernel(memory_chain_kernel, dim3((plane + 255) / 256, heads, sequences), dim3(256),
                    static_cast<size_t>(a.max_chunks) * sizeof(float), stream, a.gates,
                    a.seq_of_token, a.state_slot, static_cast<const float*>(a.state), a.chunk_state, a.tokens, a.chunk,
                    a.max_chunks, a.lay);
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(launch_kernel(memory_recurrence_kernel<T, 3>, dim3(col_blocks, heads * a.max_chunks, sequences),
                                        dim3(th), 0, stream, a));
}

}  // namespace rl

using namespace rl;

extern "C" {

enum { RL_F32 = 0, RL_BF16 = 1 };

// Floats of one request's state for `heads` heads with values of `dv` entries.
long long rl_memory_state_floats(int heads, int dv) {
  MemoryLayout lay{heads, dv};
  return static_cast<long long>(lay.slot_floats());
}

int rl_memory_gates(float* gates, const float* bias_i, const float* bias_f, float cap, const int32_t* seq_of_token,
                    const int32_t* state_slot, float* state, float* stab, int tokens, int sequences, int heads, int dv,
                    cudaStream_t stream) {
  if (tokens <= 0 || sequences <= 0) return 0;
  MemoryLayout lay{heads, dv};
  launch_kernel(memory_gates_kernel, dim3(heads, sequences), dim3(kGateThreads), 0, stream, gates, bias_i, bias_f, cap,
                seq_of_token, state_slot, state, stab, tokens, lay);
  RL_LAUNCH_END();
}

int rl_memory_recurrence(int dtype, const void* qkv, int ld, int q_col, int k_col, int v_col, float q_scale,
                         const float* gates, const int32_t* seq_of_token, const int32_t* state_slot, float* state,
                         float* num, float* qn, float* chunk_state, int tokens, int sequences, int heads, int dv,
                         int chunk, int max_chunks, cudaStream_t stream) {
  if (tokens <= 0 || sequences <= 0) return 0;
#define RL_CASE(T)                                                                                  \
  do {                                                                                              \
    MemoryArgs<T> a;                                                                                \
    a.qkv = static_cast<const T*>(qkv);                                                             \
    a.ld = ld; a.q_col = q_col; a.k_col = k_col; a.v_col = v_col; a.q_scale = q_scale;              \
    a.gates = gates; a.seq_of_token = seq_of_token; a.state_slot = state_slot; a.state = state;     \
    a.num = num; a.qn = qn; a.chunk_state = chunk_state; a.tokens = tokens; a.chunk = chunk;        \
    a.max_chunks = max_chunks; a.lay = MemoryLayout{heads, dv};                                     \
    return launch_recurrence<T>(a, sequences, stream);                                              \
  } while (0)
  if (dtype == RL_F32) RL_CASE(float);
  else RL_CASE(bf16);
#undef RL_CASE
}

int rl_memory_output(const float* num, const float* qn, const float* stab, const void* gate, int ld_gate,
                     const void* w, int w_dtype, void* out, int ld_out, int act_dtype, int tokens, int heads, int dv,
                     float eps, float floor, float out_scale, cudaStream_t stream) {
  if (tokens <= 0) return 0;
#define RL_CASE(TA, TW)                                                                                          \
  launch_kernel(memory_output_kernel<TA, TW>, dim3(tokens, (heads + 3) / 4), dim3(128), 0, stream, num, qn, stab, \
                static_cast<const TA*>(gate), ld_gate, static_cast<const TW*>(w), static_cast<TA*>(out), ld_out, \
                heads, dv, eps, floor, out_scale)
  if (act_dtype == RL_F32) RL_CASE(float, float);
  else if (w_dtype == RL_F32) RL_CASE(bf16, float);
  else RL_CASE(bf16, bf16);
#undef RL_CASE
  RL_LAUNCH_END();
}

}  // extern "C"
