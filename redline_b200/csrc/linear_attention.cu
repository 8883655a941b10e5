// Linear attention with a per-head decay, as a recurrence over a state kept per request:
//
//   S_t = decay_h * S_(t-1) + k_t v_t^T        S is [D, DV] float32 per head
//   o_t = S_t^T q_t
//
// One kernel serves prompt portions and single tokens: a CTA takes one sequence of the step, one
// head and a block of up to 128 value columns; thread j keeps column j of S (D floats) in
// registers, reads the state from the request's slot at the start and writes it back at the end.
// Columns are independent, so a head's columns may be spread over several CTAs.  A sequence's
// tokens are contiguous and in order in a step; the CTA finds them by searching the step's
// token -> sequence map.  q, k and v are read from the projection buffer in the activation type;
// the state, the decay and the sums are float32; o is written in float32.
//
// Long portions are cut in three passes so that a sequence is not one serial chain: (1) every
// chunk of C tokens sums its own contribution to the state from zero, (2) the chunks' states are
// chained (S_c = decay^C S_(c-1) + dS_c), (3) every chunk replays its tokens from its starting
// state.  A chunk's starting state is rounded no differently from the serial recurrence's except
// in the order of the sums.
#include "common.cuh"

#ifndef RL_LIN_DIM
#error "compile with -DRL_LIN_DIM=<key size>"
#endif

namespace rl {

constexpr int kD = RL_LIN_DIM;
static_assert(kD >= 1 && kD <= 256, "key size out of range");
constexpr int kTok = 16;          // tokens staged in shared memory at a time

template <typename T>
struct LinArgs {
  const T* qkv;           // [tokens, ld]: q at q_col + h * D, k at k_col + h * D, v at v_col + h * DV
  int ld, q_col, k_col, v_col;
  const int32_t* seq_of_token;   // [tokens]
  const int32_t* state_slot;     // [sequences]
  const float* decay;            // [heads]
  float* state;                  // [slots, heads, D, DV]
  float* out;                    // [tokens, heads * DV]
  float* chunk_state;            // [sequences, chunks, heads, D, DV] (chunked passes only)
  int tokens, heads, dv, chunk, max_chunks;
};

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

// mode 0: the whole sequence serially from the slot's state (state written back)
// mode 1: chunk c from zero, no outputs; the chunk's state goes to chunk_state[seq][c]
// mode 3: chunk c from its starting state as pass 2 left it (chunk_state[seq][c - 1]: the state after chunk
//         c - 1; for c = 0 the slot's state, which pass 2 has copied to the entry of the last chunk, since
//         the last chunk's CTA overwrites the slot), outputs written; the last chunk writes the slot
template <typename T, int MODE>
__global__ void __launch_bounds__(128)
linear_attention_kernel(const LinArgs<T> a) {
  pdl_launch();
  pdl_wait();
  __shared__ float qs[kTok][kD];
  __shared__ float ks[kTok][kD];
  const int seq = blockIdx.z, head = blockIdx.y % a.heads, c = blockIdx.y / a.heads;
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  const bool mine = col < a.dv;
  const int t_begin = first_token_of(a.seq_of_token, a.tokens, seq);
  const int t_end = first_token_of(a.seq_of_token, a.tokens, seq + 1);
  int t0 = t_begin, t1 = t_end;
  if (MODE != 0) {
    t0 = t_begin + c * a.chunk;
    t1 = min(t_end, t0 + a.chunk);
    if (t0 >= t_end) return;
  }
  const bool last_chunk = t1 == t_end;
  if (MODE == 1 && last_chunk) return;             // nobody starts from the state after the last chunk
  const float decay = a.decay[head];
  const int slot = a.state_slot[seq];
  const size_t plane = static_cast<size_t>(kD) * a.dv;
  float* slot_state = a.state + (static_cast<size_t>(slot) * a.heads + head) * plane;
  float* chunk_state = a.chunk_state == nullptr ? nullptr
      : a.chunk_state + ((static_cast<size_t>(seq) * a.max_chunks + c) * a.heads + head) * plane;

  float S[kD];
  if (MODE == 1) {
#pragma unroll
    for (int i = 0; i < kD; ++i) S[i] = 0.f;
  } else {
    const float* from = slot_state;
    if (MODE == 3 && c > 0) from = chunk_state - static_cast<size_t>(a.heads) * plane;
    else if (MODE == 3 && !last_chunk) {
      const int chunks = (t_end - t_begin + a.chunk - 1) / a.chunk;
      from = chunk_state + static_cast<size_t>(chunks - 1) * a.heads * plane;
    }
#pragma unroll
    for (int i = 0; i < kD; ++i) S[i] = mine ? from[static_cast<size_t>(i) * a.dv + col] : 0.f;
  }

  for (int tb = t0; tb < t1; tb += kTok) {
    const int nt = min(kTok, t1 - tb);
    __syncthreads();
    for (int i = threadIdx.x; i < nt * kD; i += blockDim.x) {
      const int tt = i / kD, d = i - tt * kD;
      const T* row = a.qkv + static_cast<size_t>(tb + tt) * a.ld;
      if (MODE != 1) qs[tt][d] = to_float(row[a.q_col + head * kD + d]);
      ks[tt][d] = to_float(row[a.k_col + head * kD + d]);
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float v = mine ? to_float(a.qkv[static_cast<size_t>(tb + tt) * a.ld + a.v_col + head * a.dv + col]) : 0.f;
      float o = 0.f;
#pragma unroll
      for (int i = 0; i < kD; ++i) {
        S[i] = fmaf(decay, S[i], ks[tt][i] * v);
        if (MODE != 1) o = fmaf(S[i], qs[tt][i], o);
      }
      if (MODE != 1 && mine) a.out[static_cast<size_t>(tb + tt) * (a.heads * a.dv) + head * a.dv + col] = o;
    }
  }
  if (!mine) return;
  float* to = MODE == 1 ? chunk_state : ((MODE == 0 || last_chunk) ? slot_state : nullptr);
  if (to != nullptr) {
#pragma unroll
    for (int i = 0; i < kD; ++i) to[static_cast<size_t>(i) * a.dv + col] = S[i];
  }
}

// Pass 2: chunk_state[seq][c] <- decay^n(c) * (state after chunk c - 1) + chunk_state[seq][c], in order of c;
// n(c) is the number of tokens of chunk c.  One thread per element of a head's state.
__global__ void linear_attention_chain_kernel(const int32_t* __restrict__ seq_of_token,
                                              const int32_t* __restrict__ state_slot, const float* __restrict__ decay,
                                              const float* __restrict__ state, float* __restrict__ chunk_state,
                                              int tokens, int heads, int dv, int chunk, int max_chunks) {
  pdl_launch();
  pdl_wait();
  const int seq = blockIdx.z, head = blockIdx.y;
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  const size_t plane = static_cast<size_t>(kD) * dv;
  if (e >= plane) return;
  const int t_begin = first_token_of(seq_of_token, tokens, seq);
  const int t_end = first_token_of(seq_of_token, tokens, seq + 1);
  const int n = t_end - t_begin;
  const int chunks = (n + chunk - 1) / chunk;
  float prev = state[(static_cast<size_t>(state_slot[seq]) * heads + head) * plane + e];
  if (chunks >= 2)     // the starting state of chunk 0, kept where no chunk's own sum lies
    chunk_state[((static_cast<size_t>(seq) * max_chunks + chunks - 1) * heads + head) * plane + e] = prev;
  float dpow = 1.f;                      // decay^chunk by repeated multiplication, as the recurrence applies it
  const float dc = decay[head];
  for (int i = 0; i < chunk; ++i) dpow *= dc;
  for (int c = 0; c + 1 < chunks; ++c) {
    float* p = chunk_state + ((static_cast<size_t>(seq) * max_chunks + c) * heads + head) * plane + e;
    prev = fmaf(dpow, prev, *p);
    *p = prev;
  }
}

template <typename T>
int launch_linear_attention(const void* qkv, int ld, int q_col, int k_col, int v_col, const int32_t* seq_of_token,
                            const int32_t* state_slot, const float* decay, float* state, float* out,
                            float* chunk_state, int tokens, int sequences, int heads, int dv, int chunk,
                            int max_chunks, cudaStream_t stream) {
  LinArgs<T> a;
  a.qkv = static_cast<const T*>(qkv);
  a.ld = ld;
  a.q_col = q_col;
  a.k_col = k_col;
  a.v_col = v_col;
  a.seq_of_token = seq_of_token;
  a.state_slot = state_slot;
  a.decay = decay;
  a.state = state;
  a.out = out;
  a.chunk_state = chunk_state;
  a.tokens = tokens;
  a.heads = heads;
  a.dv = dv;
  a.chunk = chunk;
  a.max_chunks = max_chunks;
  const int th = dv >= 128 ? 128 : (dv + 31) / 32 * 32;
  const int col_blocks = (dv + th - 1) / th;
  if (chunk_state == nullptr || max_chunks <= 1) {
    return static_cast<int>(launch_kernel(linear_attention_kernel<T, 0>, dim3(col_blocks, heads, sequences), dim3(th),
                                          0, stream, a));
  }
  cudaError_t e = launch_kernel(linear_attention_kernel<T, 1>, dim3(col_blocks, heads * max_chunks, sequences),
                                dim3(th), 0, stream, a);
  if (e != cudaSuccess) return static_cast<int>(e);
  const int plane = kD * dv;
  e = launch_kernel(linear_attention_chain_kernel, dim3((plane + 255) / 256, heads, sequences), dim3(256), 0, stream,
                    seq_of_token, state_slot, decay, static_cast<const float*>(state), chunk_state, tokens, heads, dv,
                    chunk, max_chunks);
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(launch_kernel(linear_attention_kernel<T, 3>, dim3(col_blocks, heads * max_chunks, sequences),
                                        dim3(th), 0, stream, a));
}

}  // namespace rl

using namespace rl;

extern "C" {

// chunk_state null or max_chunks <= 1: every sequence is one serial chain.  Otherwise sequences are cut
// into chunks of `chunk` tokens (max_chunks = the most chunks any sequence of the step has) and
// chunk_state holds [sequences, max_chunks, heads, D, DV] floats.
int rl_linear_attention(int dtype, const void* qkv, int ld, int q_col, int k_col, int v_col,
                        const int32_t* seq_of_token, const int32_t* state_slot, const float* decay, float* state,
                        float* out, float* chunk_state, int tokens, int sequences, int heads, int dv, int chunk,
                        int max_chunks, cudaStream_t stream) {
  if (tokens <= 0 || sequences <= 0) return 0;
  if (dtype == 0)
    return launch_linear_attention<float>(qkv, ld, q_col, k_col, v_col, seq_of_token, state_slot, decay, state, out,
                                          chunk_state, tokens, sequences, heads, dv, chunk, max_chunks, stream);
  return launch_linear_attention<bf16>(qkv, ld, q_col, k_col, v_col, seq_of_token, state_slot, decay, state, out,
                                       chunk_state, tokens, sequences, heads, dv, chunk, max_chunks, stream);
}

}  // extern "C"
