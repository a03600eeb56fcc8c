// Mixers that carry a state of fixed size from token to token: a short causal
// convolution over time, a selective state space with one decay per head
// (Mamba-2's recurrence), the gated delta rule, and the gated norm behind both.
//
// Everything that enters a recurrence is float32 whatever the activation type:
// step sizes (softplus), decays (exp), gates (sigmoid), unit norms and the state
// itself.  A request's tokens are taken in order; a segment of a step continues
// from the state its request's slot holds and leaves the state there.  A token's
// result depends on its own request alone: on nothing else in the launch, and on
// how the request was cut into steps only through float32 rounding (it is not:
// every token performs the same operations in the same order whatever the cut).
//
//   conv_silu        y[t,c] = silu(b_c + sum_j w[c,j] u[t-(taps-1)+j, c]); the last
//                    taps-1 inputs of a request live in its state slot
//   ssd_scan         S <- exp(-exp(A) dt) S + dt B x^T ; y = S^T C + D x       (S: N x P per head)
//   delta_scan       S <- g S ; u = beta (v - S^T k) ; S <- S + k u^T ; o = S^T q   (S: D x P per head)
//   gated_norm       rms over groups of a row, a gate silu(z) before or after it
//
// State layout per head: [N or D][P] float32, P contiguous.  A warp owns WC
// columns of a head's state and its lanes split the rows, so a column's dot
// products are one warp reduction; a block's four warps share the tokens of a
// chunk, which all threads stage into shared memory together.  Which WC a launch
// takes depends on the step's shape, never on a token's place in it, and the
// operations on a column are the same for every WC.
#include "common.cuh"

namespace ft {

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }
// a gate's function: 0 silu, 1 sigmoid
__device__ __forceinline__ float gate_f(float v, int kind) {
  const float sg = 1.f / (1.f + expf(-v));
  return kind == 1 ? sg : v * sg;
}

// Sums V values per lane over the warp with V - 1 + log2(32 / V) shuffles: at every step a lane
// hands half of its values to the lane `mask` away and adds what it gets to the half it keeps.
// Afterwards v[0] of lane l is the warp's total of value  l >> (5 - log2 V).
template <int V>
__device__ __forceinline__ void warp_sum_multi(float (&v)[V]) {
  const int lane = threadIdx.x & 31;
  int mask = 16;
#pragma unroll
  for (int w = V / 2; w >= 1; w >>= 1) {
    const bool upper = lane & mask;
#pragma unroll
    for (int i = 0; i < w; ++i) {
      const float send = upper ? v[i] : v[i + w];
      const float keep = upper ? v[i + w] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, mask);
    }
    mask >>= 1;
  }
  for (; mask >= 1; mask >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], mask);
}
template <int V> struct Log2 { static constexpr int value = 1 + Log2<V / 2>::value; };
template <> struct Log2<1> { static constexpr int value = 0; };

// ------------------------------------------------------------ short convolution
struct ConvArgs {
  const void* x;        // [T, ldx]: channel c of token t at x[t * ldx + c]
  void* out;            // [T, ldo]
  const float* w;       // [C, taps]; the last column weighs the current token
  const float* bias;    // [C] or nullptr
  float* state;         // slot s: state + s * slot_stride, [taps - 1][C], oldest input first
  const int* token_seg; // [T]
  const int* seg_slot;  // [S]
  const int* seg_q_start;  // [S + 1]
  long long ldx, ldo, slot_stride;
  int C, taps;
  int act;              // 1: SiLU behind the sum; 0: the sum itself
};

constexpr int CONV_MAX_TAPS = 8;     // longer convolutions take the plain loop

// A thread owns one channel (two neighbouring ones where rows allow 4-byte pieces of bfloat16)
// and `run` consecutive tokens: while they belong to one segment it keeps the last taps inputs
// in registers and fetches one new input a token; at a segment's first token (and always when
// run is 1) it fetches the whole reach, from earlier rows or from the slot.  The sum runs over
// ascending taps either way.
template <typename AT, int CPT, int RUN>
__global__ void __launch_bounds__(128) conv_silu_kernel(ConvArgs a, int T) {
  constexpr int run = RUN;
  pdl_wait();
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * CPT;
  if (c >= a.C) return;
  const int K = a.taps - 1;
  const AT* x = (const AT*)a.x;
  float w[CPT][CONV_MAX_TAPS], win[CPT][CONV_MAX_TAPS], bias[CPT];
#pragma unroll
  for (int u = 0; u < CPT; ++u) {
    bias[u] = a.bias ? a.bias[c + u] : 0.f;
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) w[u][j] = j <= K ? a.w[(size_t)(c + u) * a.taps + j] : 0.f;
  }
  auto fetch = [&](int row, float (&v)[CPT]) {          // CPT inputs of a token's row
    if constexpr (CPT == 2) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + (size_t)row * a.ldx + c));
      v[0] = f.x;
      v[1] = f.y;
    } else {
      v[0] = to_float(x[(size_t)row * a.ldx + c]);
    }
  };
  int prev_seg = -1;
  const int t_first = blockIdx.x * run, t_end = min(T, (blockIdx.x + 1) * run);
  // every token's own input and segment first, all loads in flight together
  float own[RUN][CPT];
  int segs[RUN];
#pragma unroll
  for (int i = 0; i < RUN; ++i) {
    if (t_first + i < t_end) {
      fetch(t_first + i, own[i]);
      segs[i] = a.token_seg[t_first + i];
    }
  }
#pragma unroll
  for (int i = 0; i < RUN; ++i) {
    const int t = t_first + i;
    if (t >= t_end) break;
    const int seg = segs[i];
    const int q0 = a.seg_q_start[seg];
    const int r = t - q0;
    if (seg != prev_seg) {
      const float* st = a.state + (size_t)a.seg_slot[seg] * a.slot_stride;
#pragma unroll
      for (int j = 0; j < CONV_MAX_TAPS; ++j) {
        if (j > K) break;
        const int s = r - K + j;
        float v[CPT];
        if (s == r) {
#pragma unroll
          for (int u = 0; u < CPT; ++u) v[u] = own[i][u];
        } else if (s >= 0) fetch(q0 + s, v);
        else {
#pragma unroll
          for (int u = 0; u < CPT; ++u) v[u] = st[(size_t)(K + s) * a.C + c + u];
        }
#pragma unroll
        for (int u = 0; u < CPT; ++u) win[u][j] = v[u];
      }
      prev_seg = seg;
    } else {
#pragma unroll
      for (int u = 0; u < CPT; ++u) {
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS - 1; ++j)
          if (j < K) win[u][j] = win[u][j + 1];
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; ++j)
          if (j == K) win[u][j] = own[i][u];
      }
    }
    float out[CPT];
#pragma unroll
    for (int u = 0; u < CPT; ++u) {
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < CONV_MAX_TAPS; ++j)
        if (j <= K) acc = fmaf(w[u][j], win[u][j], acc);
      out[u] = a.act ? silu_f(acc + bias[u]) : acc + bias[u];
    }
    AT* o = (AT*)a.out + (size_t)t * a.ldo + c;
    if constexpr (CPT == 2) *reinterpret_cast<__nv_bfloat162*>(o) = __floats2bfloat162_rn(out[0], out[1]);
    else o[0] = from_float<AT>(out[0]);
  }
}

// any number of taps: one channel and one token a thread
template <typename AT>
__global__ void __launch_bounds__(128) conv_silu_long_kernel(ConvArgs a) {
  pdl_wait();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= a.C) return;
  const int seg = a.token_seg[t];
  const int q0 = a.seg_q_start[seg];
  const int r = t - q0, K = a.taps - 1;
  const float* st = a.state + (size_t)a.seg_slot[seg] * a.slot_stride;
  const AT* x = (const AT*)a.x;
  float acc = 0.f;
  for (int j = 0; j <= K; ++j) {
    const int s = r - K + j;
    const float v = s >= 0 ? to_float(x[(size_t)(q0 + s) * a.ldx + c]) : st[(size_t)(K + s) * a.C + c];
    acc = fmaf(a.w[(size_t)c * a.taps + j], v, acc);
  }
  if (a.bias) acc += a.bias[c];
  ((AT*)a.out)[(size_t)t * a.ldo + c] = from_float<AT>(a.act ? silu_f(acc) : acc);
}

// After the convolution has read it: the slot keeps the last taps-1 inputs of (what it held ++
// the segment's inputs).  Ascending i reads entries at or above the one it writes.
template <typename AT>
__global__ void __launch_bounds__(128) conv_state_kernel(ConvArgs a) {
  pdl_wait();
  const int seg = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= a.C) return;
  const int q0 = a.seg_q_start[seg], n = a.seg_q_start[seg + 1] - q0, K = a.taps - 1;
  float* st = a.state + (size_t)a.seg_slot[seg] * a.slot_stride;
  const AT* x = (const AT*)a.x;
  for (int i = 0; i < K; ++i) {
    const int src = n + i;
    st[(size_t)i * a.C + c] = src < K ? st[(size_t)src * a.C + c] : to_float(x[(size_t)(q0 + src - K) * a.ldx + c]);
  }
}

// -------------------------------------------------------- selective state space
// Both scans share their shape.  A block of four warps owns COLS = 4 * WC columns of one head's
// state in one segment; a warp owns WC of them and its lanes split the rows (NPL rows a lane).
// Tokens come in chunks of SCAN_CHUNK: every thread fetches its share of the NEXT chunk's rows
// into registers before the block works through the current chunk from shared memory, and puts
// them into the other of two buffers afterwards, so that the loads' latency hides under the
// arithmetic and a chunk costs one block-wide barrier.  A full chunk's tokens are unrolled, so
// that the shuffles of one token's read-out overlap the next token's products.
constexpr int SCAN_WARPS = 4;
constexpr int SCAN_THREADS = SCAN_WARPS * 32;
constexpr int SCAN_CHUNK = 8;

// WC consecutive floats of a state row: 16- or 8-byte pieces when `vec` says they are aligned
template <int WC>
__device__ __forceinline__ void load_cols(const float* p, float (&v)[WC], int valid, bool vec) {
  if (WC > 1 && vec && valid >= WC) {
    if constexpr (WC % 4 == 0) {
#pragma unroll
      for (int c = 0; c < WC; c += 4) {
        const float4 f = *reinterpret_cast<const float4*>(p + c);
        v[c] = f.x; v[c + 1] = f.y; v[c + 2] = f.z; v[c + 3] = f.w;
      }
    } else if constexpr (WC % 2 == 0) {
#pragma unroll
      for (int c = 0; c < WC; c += 2) {
        const float2 f = *reinterpret_cast<const float2*>(p + c);
        v[c] = f.x; v[c + 1] = f.y;
      }
    }
    return;
  }
#pragma unroll
  for (int c = 0; c < WC; ++c) v[c] = c < valid ? p[c] : 0.f;
}
template <int WC>
__device__ __forceinline__ void store_cols(float* p, const float (&v)[WC], int valid, bool vec) {
  if (WC > 1 && vec && valid >= WC) {
    if constexpr (WC % 4 == 0) {
#pragma unroll
      for (int c = 0; c < WC; c += 4) *reinterpret_cast<float4*>(p + c) = make_float4(v[c], v[c + 1], v[c + 2], v[c + 3]);
    } else if constexpr (WC % 2 == 0) {
#pragma unroll
      for (int c = 0; c < WC; c += 2) *reinterpret_cast<float2*>(p + c) = make_float2(v[c], v[c + 1]);
    }
    return;
  }
#pragma unroll
  for (int c = 0; c < WC; ++c)
    if (c < valid) p[c] = v[c];
}

struct SsdArgs {
  const void* xbc;      // [T, ld]: x (heads * P) | B (G * N) | C (G * N), after convolution and silu
  const void* dt;       // [T, ld_dt]: the step size's projection, head h at column h
  const float* dt_bias; // [heads]
  const float* A_log;   // [heads]
  const float* D;       // [heads]
  float* state;         // slot s: state + s * slot_stride, [heads][N][P]
  float* y;             // [T, heads * P] float32
  const int* seg_slot;
  const int* seg_q_start;
  long long ld, ld_dt, slot_stride;
  int heads, P, N, G;
  int vec;              // state rows may be read in 16-byte (WC % 4 == 0) or 8-byte pieces
};

// NPL: state rows a lane holds (N <= 32 * NPL); WC: state columns a warp owns
template <typename AT, int NPL, int WC>
__global__ void __launch_bounds__(SCAN_THREADS) ssd_scan_kernel(SsdArgs a) {
  constexpr int COLS = SCAN_WARPS * WC;
  constexpr int NB = (NPL * 32 + SCAN_THREADS - 1) / SCAN_THREADS;       // B (or C) values a thread stages per token
  constexpr int XR = (SCAN_CHUNK * COLS + SCAN_THREADS - 1) / SCAN_THREADS;
  extern __shared__ float sm[];
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int head = blockIdx.y, seg = blockIdx.z;
  const int N = a.N, P = a.P;
  const int g = head / (a.heads / a.G);
  const int inner = a.heads * P;
  const int col0 = blockIdx.x * COLS;
  const int j0 = col0 + warp * WC;
  const int per = SCAN_CHUNK * (2 * N + COLS + 2);                         // floats of one buffer
  const int q0 = a.seg_q_start[seg], q1 = a.seg_q_start[seg + 1];
  float* st = a.state + (size_t)a.seg_slot[seg] * a.slot_stride + (size_t)head * N * P;
  const float rate = -expf(a.A_log[head]), bias = a.dt_bias[head], skip = a.D[head];
  const AT* xbc = (const AT*)a.xbc;
  const AT* dt = (const AT*)a.dt;

  float S[NPL][WC];
#pragma unroll
  for (int e = 0; e < NPL; ++e) {
    const int n = lane + 32 * e;
    if (n < N) load_cols<WC>(st + (size_t)n * P + j0, S[e], P - j0, a.vec);
    else {
#pragma unroll
      for (int c = 0; c < WC; ++c) S[e][c] = 0.f;
    }
  }

  AT pb[SCAN_CHUNK][NB], pc[SCAN_CHUNK][NB], px[XR], pdt;
  auto fetch = [&](int t0, int nt) {
#pragma unroll
    for (int tt = 0; tt < SCAN_CHUNK; ++tt) {
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const int n = threadIdx.x + SCAN_THREADS * b;
        if (tt < nt && n < N) {
          const AT* row = xbc + (size_t)(t0 + tt) * a.ld + inner + (size_t)g * N + n;
          pb[tt][b] = row[0];
          pc[tt][b] = row[(size_t)a.G * N];
        }
      }
    }
#pragma unroll
    for (int r = 0; r < XR; ++r) {
      const int i = threadIdx.x + SCAN_THREADS * r, tt = i / COLS, c = i % COLS;
      px[r] = (tt < nt && col0 + c < P) ? xbc[(size_t)(t0 + tt) * a.ld + (size_t)head * P + col0 + c] : from_float<AT>(0.f);
    }
    if ((int)threadIdx.x < nt) pdt = dt[(size_t)(t0 + threadIdx.x) * a.ld_dt + head];
  };
  auto put = [&](float* buf, int nt) {
    float* Bs = buf;
    float* Cs = Bs + SCAN_CHUNK * N;
    float* xs = Cs + SCAN_CHUNK * N;
    float* dts = xs + SCAN_CHUNK * COLS;
#pragma unroll
    for (int tt = 0; tt < SCAN_CHUNK; ++tt) {
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const int n = threadIdx.x + SCAN_THREADS * b;
        if (tt < nt && n < N) {
          Bs[tt * N + n] = to_float(pb[tt][b]);
          Cs[tt * N + n] = to_float(pc[tt][b]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < XR; ++r) {
      const int i = threadIdx.x + SCAN_THREADS * r;
      if (i < SCAN_CHUNK * COLS) xs[i] = to_float(px[r]);
    }
    if ((int)threadIdx.x < nt) {
      const float step = softplus_f(to_float(pdt) + bias);
      dts[threadIdx.x] = step;
      dts[SCAN_CHUNK + threadIdx.x] = expf(rate * step);
    }
  };

  fetch(q0, min(SCAN_CHUNK, q1 - q0));
  put(sm, min(SCAN_CHUNK, q1 - q0));
  __syncthreads();
  int turn = 0;
  for (int t0 = q0; t0 < q1; t0 += SCAN_CHUNK, turn ^= 1) {
    const int nt = min(SCAN_CHUNK, q1 - t0);
    const int next = min(SCAN_CHUNK, q1 - t0 - SCAN_CHUNK);
    if (next > 0) fetch(t0 + SCAN_CHUNK, next);
    const float* Bs = sm + turn * per;
    const float* Cs = Bs + SCAN_CHUNK * N;
    const float* xs = Cs + SCAN_CHUNK * N;
    const float* dts = xs + SCAN_CHUNK * COLS;
    auto token = [&](int tt) {
      const float step = dts[tt], decay = dts[SCAN_CHUNK + tt];
      float Bv[NPL], Cv[NPL];
#pragma unroll
      for (int e = 0; e < NPL; ++e) {
        const int n = lane + 32 * e;
        Bv[e] = n < N ? Bs[tt * N + n] : 0.f;
        Cv[e] = n < N ? Cs[tt * N + n] : 0.f;
      }
      float part[WC], xv[WC];
#pragma unroll
      for (int c = 0; c < WC; ++c) {
        xv[c] = xs[tt * COLS + warp * WC + c];
        const float in = step * xv[c];
        float acc = 0.f;
#pragma unroll
        for (int e = 0; e < NPL; ++e) {
          S[e][c] = fmaf(decay, S[e][c], in * Bv[e]);
          acc = fmaf(S[e][c], Cv[e], acc);
        }
        part[c] = acc;
      }
      warp_sum_multi<WC>(part);
      const int c = lane >> (5 - Log2<WC>::value);
      if ((lane & ((32 / WC) - 1)) == 0 && j0 + c < P) {
        float mine = xv[0];
#pragma unroll
        for (int i = 1; i < WC; ++i) mine = c == i ? xv[i] : mine;
        a.y[(size_t)(t0 + tt) * inner + (size_t)head * P + j0 + c] = part[0] + skip * mine;
      }
    };
    if (nt == SCAN_CHUNK) {
#pragma unroll
      for (int tt = 0; tt < SCAN_CHUNK; ++tt) token(tt);
    } else {
      for (int tt = 0; tt < nt; ++tt) token(tt);
    }
    if (next > 0) put(sm + (turn ^ 1) * per, next);
    __syncthreads();
  }
#pragma unroll
  for (int e = 0; e < NPL; ++e) {
    const int n = lane + 32 * e;
    if (n < N) store_cols<WC>(st + (size_t)n * P + j0, S[e], P - j0, a.vec);
  }
}

// ------------------------------------------------------------- gated delta rule
struct DeltaArgs {
  const void* qkv;      // [T, ld]: q (G * D) | k (G * D) | v (heads * P), after convolution and silu
  const void* beta;     // [T, ld_gate]: the write strength's projection, head h at column h
  const void* decay;    // [T, ld_gate]: the decay's projection, head h at column h
  const float* dt_bias; // [heads]
  const float* A_log;   // [heads]
  float* state;         // slot s: state + s * slot_stride, [heads][D][P]
  float* o;             // [T, heads * P] float32
  const int* seg_slot;
  const int* seg_q_start;
  long long ld, ld_gate, slot_stride;
  int heads, P, D, G;
  float unit_eps, q_scale;
  int vec;
  // MODE 1: a decay per key channel
  const float* decay_rows;   // [T, ld_decay] float32: the decay's projection, channel n of head h at h * D + n;
  long long ld_decay;        // dt_bias is then [heads * D]
  // MODE 2: retention
  const float* cos_sin;      // [positions, rot_dims]: cos | sin (nullptr or rot_dims 0: no rotation)
  const int* seg_pos0;       // [S]: position of a segment's first token
  int rot_dims;
};

// MODE 0: the gated delta rule with one decay per head.
// MODE 1: the same rule with a decay per key channel: row n of a head's state is multiplied by
//         g_n = exp(-exp(A_log_h) softplus(a_n + dt_bias[h * D + n])) before the token reads and writes.
// MODE 2: retention: S <- c_h S + k v^T, o = S^T q with a constant c_h per head (dt_bias[h]), no write
//         strength and no unit norms; q and k have the first rot_dims dimensions of each head turned
//         by the token's position (dimension i with i + rot_dims / 2) in shared memory, in float32;
//         k is multiplied by q_scale after the rotation.
template <typename AT, int NPL, int WC, int MODE>
__global__ void __launch_bounds__(SCAN_THREADS) delta_scan_kernel(DeltaArgs a) {
  constexpr int COLS = SCAN_WARPS * WC;
  constexpr int NB = (NPL * 32 + SCAN_THREADS - 1) / SCAN_THREADS;
  constexpr int XR = (SCAN_CHUNK * COLS + SCAN_THREADS - 1) / SCAN_THREADS;
  extern __shared__ float sm[];
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int head = blockIdx.y, seg = blockIdx.z;
  const int D = a.D, P = a.P;
  const int g = head / (a.heads / a.G);
  const int col0 = blockIdx.x * COLS;
  const int j0 = col0 + warp * WC;
  const int width = a.heads * P;
  const int per = SCAN_CHUNK * ((MODE == 1 ? 3 : 2) * D + COLS + 2);
  const int q0 = a.seg_q_start[seg], q1 = a.seg_q_start[seg + 1];
  float* st = a.state + (size_t)a.seg_slot[seg] * a.slot_stride + (size_t)head * D * P;
  const float rate = MODE == 2 ? 0.f : -expf(a.A_log[head]);
  const float bias = MODE == 1 ? 0.f : a.dt_bias[head];      // MODE 2: the head's constant decay
  const AT* qkv = (const AT*)a.qkv;
  const int half = MODE == 2 ? a.rot_dims >> 1 : 0;
  const int pos0 = MODE == 2 && half ? a.seg_pos0[seg] : 0;
  float ch_bias[NB];                                          // MODE 1: dt_bias of this thread's channels
  if constexpr (MODE == 1) {
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      const int n = threadIdx.x + SCAN_THREADS * b;
      ch_bias[b] = n < D ? a.dt_bias[(size_t)head * D + n] : 0.f;
    }
  }

  float S[NPL][WC];
#pragma unroll
  for (int e = 0; e < NPL; ++e) {
    const int n = lane + 32 * e;
    if (n < D) load_cols<WC>(st + (size_t)n * P + j0, S[e], P - j0, a.vec);
    else {
#pragma unroll
      for (int c = 0; c < WC; ++c) S[e][c] = 0.f;
    }
  }

  AT pq[SCAN_CHUNK][NB], pk[SCAN_CHUNK][NB], pv[XR], pbeta, pdecay;
  float pg[MODE == 1 ? SCAN_CHUNK : 1][NB];                   // MODE 1: the channels' decay projections
  float pcos[MODE == 2 ? NPL : 1], psin[MODE == 2 ? NPL : 1]; // MODE 2: pair (tt, i) = threadIdx.x + 128 r
  auto fetch = [&](int t0, int nt) {
#pragma unroll
    for (int tt = 0; tt < SCAN_CHUNK; ++tt) {
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const int n = threadIdx.x + SCAN_THREADS * b;
        if (tt < nt && n < D) {
          const AT* row = qkv + (size_t)(t0 + tt) * a.ld + (size_t)g * D + n;
          pq[tt][b] = row[0];
          pk[tt][b] = row[(size_t)a.G * D];
          if constexpr (MODE == 1) pg[tt][b] = a.decay_rows[(size_t)(t0 + tt) * a.ld_decay + (size_t)head * D + n];
        }
      }
    }
    if constexpr (MODE == 2) {
#pragma unroll
      for (int r = 0; r < NPL; ++r) {
        const int idx = threadIdx.x + SCAN_THREADS * r;
        if (half && idx < nt * half) {
          const int tt = idx / half, i = idx - tt * half;
          const float* cs = a.cos_sin + (size_t)(pos0 + t0 + tt - q0) * a.rot_dims;
          pcos[r] = cs[i];
          psin[r] = cs[half + i];
        }
      }
    }
#pragma unroll
    for (int r = 0; r < XR; ++r) {
      const int i = threadIdx.x + SCAN_THREADS * r, tt = i / COLS, c = i % COLS;
      pv[r] = (tt < nt && col0 + c < P)
                  ? qkv[(size_t)(t0 + tt) * a.ld + 2 * (size_t)a.G * D + (size_t)head * P + col0 + c]
                  : from_float<AT>(0.f);
    }
    if (MODE != 2 && (int)threadIdx.x < nt) {
      const size_t at = (size_t)(t0 + threadIdx.x) * a.ld_gate + head;
      pbeta = ((const AT*)a.beta)[at];
      if constexpr (MODE == 0) pdecay = ((const AT*)a.decay)[at];
    }
  };
  auto put = [&](float* buf, int nt) {
    float* qs = buf;
    float* ks = qs + SCAN_CHUNK * D;
    float* vs = ks + SCAN_CHUNK * D;
    float* gates = vs + SCAN_CHUNK * COLS;
#pragma unroll
    for (int tt = 0; tt < SCAN_CHUNK; ++tt) {
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const int n = threadIdx.x + SCAN_THREADS * b;
        if (tt < nt && n < D) {
          qs[tt * D + n] = to_float(pq[tt][b]);
          ks[tt * D + n] = to_float(pk[tt][b]);
          if constexpr (MODE == 1)
            gates[2 * SCAN_CHUNK + tt * D + n] = expf(rate * softplus_f(pg[tt][b] + ch_bias[b]));
        }
      }
    }
#pragma unroll
    for (int r = 0; r < XR; ++r) {
      const int i = threadIdx.x + SCAN_THREADS * r;
      if (i < SCAN_CHUNK * COLS) vs[i] = to_float(pv[r]);
    }
    if ((int)threadIdx.x < nt) {
      if constexpr (MODE == 2) {
        gates[threadIdx.x] = 1.f;
        gates[SCAN_CHUNK + threadIdx.x] = bias;
      } else {
        gates[threadIdx.x] = 1.f / (1.f + expf(-to_float(pbeta)));
        gates[SCAN_CHUNK + threadIdx.x] = MODE == 1 ? 1.f : expf(rate * softplus_f(to_float(pdecay) + bias));
      }
    }
  };
  // MODE 2: turn the staged q and k rows of a chunk; a thread owns whole pairs
  auto turn_rows = [&](float* buf, int nt) {
    if constexpr (MODE == 2) {
      float* qs = buf;
      float* ks = qs + SCAN_CHUNK * D;
#pragma unroll
      for (int r = 0; r < NPL; ++r) {
        const int idx = threadIdx.x + SCAN_THREADS * r;
        if (half && idx < nt * half) {
          const int tt = idx / half, i = idx - tt * half;
          const float c = pcos[r], sn = psin[r];
          float* qa = qs + tt * D + i;
          float* ka = ks + tt * D + i;
          const float qu = qa[0], qv = qa[half], ku = ka[0], kv_ = ka[half];
          qa[0] = qu * c - qv * sn;
          qa[half] = qv * c + qu * sn;
          ka[0] = ku * c - kv_ * sn;
          ka[half] = kv_ * c + ku * sn;
        }
      }
    }
  };

  fetch(q0, min(SCAN_CHUNK, q1 - q0));
  put(sm, min(SCAN_CHUNK, q1 - q0));
  if constexpr (MODE == 2) {
    __syncthreads();
    turn_rows(sm, min(SCAN_CHUNK, q1 - q0));
  }
  __syncthreads();
  int turn = 0;
  for (int t0 = q0; t0 < q1; t0 += SCAN_CHUNK, turn ^= 1) {
    const int nt = min(SCAN_CHUNK, q1 - t0);
    const int next = min(SCAN_CHUNK, q1 - t0 - SCAN_CHUNK);
    if (next > 0) fetch(t0 + SCAN_CHUNK, next);
    const float* qs = sm + turn * per;
    const float* ks = qs + SCAN_CHUNK * D;
    const float* vs = ks + SCAN_CHUNK * D;
    const float* gates = vs + SCAN_CHUNK * COLS;
    auto token = [&](int tt) {
      const float beta = gates[tt], decay = gates[SCAN_CHUNK + tt];
      float qv[NPL], kv[NPL];
      // sums of squares of the raw q and k rows and their product: unit vectors without a pass of
      // their own (every warp of the block forms them for itself; they do not wait for the state)
      float unit[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int e = 0; e < NPL; ++e) {
        const int n = lane + 32 * e;
        qv[e] = n < D ? qs[tt * D + n] : 0.f;
        kv[e] = n < D ? ks[tt * D + n] : 0.f;
        if constexpr (MODE == 2) kv[e] *= a.q_scale;
        unit[0] = fmaf(qv[e], qv[e], unit[0]);
        unit[1] = fmaf(kv[e], kv[e], unit[1]);
        unit[2] = fmaf(qv[e], kv[e], unit[2]);
      }
      warp_sum_multi<4>(unit);
      const float mine_u = unit[0];                       // lane l holds value l >> 3
      float kq;
      if constexpr (MODE == 2) {
        kq = __shfl_sync(0xffffffffu, mine_u, 16);
      } else {
        const float iq = a.q_scale / sqrtf(__shfl_sync(0xffffffffu, mine_u, 0) + a.unit_eps);
        const float ik = 1.f / sqrtf(__shfl_sync(0xffffffffu, mine_u, 8) + a.unit_eps);
        kq = __shfl_sync(0xffffffffu, mine_u, 16) * iq * ik;
#pragma unroll
        for (int e = 0; e < NPL; ++e) {
          qv[e] *= iq;
          kv[e] *= ik;
        }
      }
      if constexpr (MODE == 1) {
        // every row of the state decays by its own channel's factor before the token reads it
#pragma unroll
        for (int e = 0; e < NPL; ++e) {
          const int n = lane + 32 * e;
          const float gn = n < D ? gates[2 * SCAN_CHUNK + tt * D + n] : 1.f;
#pragma unroll
          for (int c = 0; c < WC; ++c) S[e][c] *= gn;
        }
      }
      // per column: S^T k and S^T q of the state before this token
      float red[2 * WC];
#pragma unroll
      for (int c = 0; c < WC; ++c) {
        float sa = 0.f, sb = 0.f;
#pragma unroll
        for (int e = 0; e < NPL; ++e) {
          sa = fmaf(S[e][c], kv[e], sa);
          sb = fmaf(S[e][c], qv[e], sb);
        }
        red[c] = sa;
        red[WC + c] = sb;
      }
      warp_sum_multi<2 * WC>(red);
      constexpr int SHIFT = 5 - Log2<2 * WC>::value;      // lane l holds the total of value l >> SHIFT
      const float mine = red[0];
#pragma unroll
      for (int c = 0; c < WC; ++c) {
        const float sa = __shfl_sync(0xffffffffu, mine, c << SHIFT);
        const float sb = __shfl_sync(0xffffffffu, mine, (WC + c) << SHIFT);
        const float v = vs[tt * COLS + warp * WC + c];
        // the decayed state answers k with decay * sa; the token writes u along k, and its own
        // read-out already contains that write: decay * sb + (k . q) u
        const float u = MODE == 2 ? v : beta * (v - decay * sa);
        if (lane == 0 && j0 + c < P)
          a.o[(size_t)(t0 + tt) * width + (size_t)head * P + j0 + c] = fmaf(kq, u, decay * sb);
#pragma unroll
        for (int e = 0; e < NPL; ++e) S[e][c] = fmaf(kv[e], u, decay * S[e][c]);
      }
    };
    if (nt == SCAN_CHUNK) {
#pragma unroll
      for (int tt = 0; tt < SCAN_CHUNK; ++tt) token(tt);
    } else {
      for (int tt = 0; tt < nt; ++tt) token(tt);
    }
    if (next > 0) put(sm + (turn ^ 1) * per, next);
    if constexpr (MODE == 2) {
      if (next > 0) {
        __syncthreads();
        turn_rows(sm + (turn ^ 1) * per, next);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int e = 0; e < NPL; ++e) {
    const int n = lane + 32 * e;
    if (n < D) store_cols<WC>(st + (size_t)n * P + j0, S[e], P - j0, a.vec);
  }
}

// --------------------------------------------------------------------- gated norm
// A row of `width` float32 values in `groups` equal parts, each divided by its own root mean
// square; times weight[i % weight_len]; a gate silu(z) (or sigmoid(z)) on the values before the norm
// (gate_first) or on the result.  One warp per (token, group).
template <typename AT>
__global__ void __launch_bounds__(128) gated_norm_kernel(const float* __restrict__ y, const AT* __restrict__ z,
                                                         long long ldz, const float* __restrict__ weight,
                                                         int weight_len, AT* __restrict__ out, int T, int width,
                                                         int groups, float eps, int gate_first, int gate_kind) {
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)T * groups) return;
  const int t = (int)(item / groups), grp = (int)(item % groups);
  const int size = width / groups, base = grp * size;
  const float* row = y + (size_t)t * width + base;
  const AT* gate = z + (size_t)t * ldz + base;
  float ss = 0.f;
  for (int i = lane; i < size; i += 32) {
    float v = row[i];
    if (gate_first) v *= gate_f(to_float(gate[i]), gate_kind);
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.f / sqrtf(warp_sum(ss) / (float)size + eps);
  AT* dst = out + (size_t)t * width + base;
  for (int i = lane; i < size; i += 32) {
    const float gv = gate_f(to_float(gate[i]), gate_kind);
    float v = row[i];
    if (gate_first) v *= gv;
    v = v * inv * weight[(base + i) % weight_len];
    if (!gate_first) v *= gv;
    dst[i] = from_float<AT>(v);
  }
}

// The same norm with TPI threads per (token, group), 16-byte pieces, and every value kept in
// registers between the sum of squares and the scaling: parts of up to 4 * KEEP * TPI values, a
// multiple of 4, rows 16-byte (bfloat16 gate: 8-byte) aligned.
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(__nv_bfloat16* p, float4 v) {
  uint2 raw;
  *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v.x, v.y);
  *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = raw;
}

template <typename AT, int TPI, int KEEP>
__global__ void __launch_bounds__(128) gated_norm_vec_kernel(const float* __restrict__ y, const AT* __restrict__ z,
                                                             long long ldz, const float* __restrict__ weight,
                                                             int weight_len, AT* __restrict__ out, int T, int width,
                                                             int groups, float eps, int gate_first, int gate_kind) {
  __shared__ float scratch[33];
  pdl_wait();
  const int sub = threadIdx.x % TPI;
  const long long item = (long long)blockIdx.x * (128 / TPI) + threadIdx.x / TPI;
  if (item >= (long long)T * groups) return;          // a warp (TPI 32) or the whole block (TPI 128) leaves
  const int t = (int)(item / groups), grp = (int)(item % groups);
  const int size = width / groups, base = grp * size, pieces = size >> 2;
  const float* row = y + (size_t)t * width + base;
  const AT* gate = z + (size_t)t * ldz + base;
  float4 keep[KEEP], gk[KEEP];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < KEEP; ++j) {
    const int gi = sub + j * TPI;
    if (gi < pieces) {
      float4 v = ld4(row + 4 * gi);
      const float4 gr = ld4(gate + 4 * gi);
      const float4 gv = make_float4(gate_f(gr.x, gate_kind), gate_f(gr.y, gate_kind), gate_f(gr.z, gate_kind), gate_f(gr.w, gate_kind));
      if (gate_first) { v.x *= gv.x; v.y *= gv.y; v.z *= gv.z; v.w *= gv.w; }
      keep[j] = v;
      gk[j] = gv;
      ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    }
  }
  ss = TPI == 32 ? warp_sum(ss) : block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)size + eps);
  AT* dst = out + (size_t)t * width + base;
#pragma unroll
  for (int j = 0; j < KEEP; ++j) {
    const int gi = sub + j * TPI;
    if (gi < pieces) {
      const float4 w = ld4(weight + (base + 4 * gi) % weight_len);
      float4 v = keep[j];
      v.x *= inv * w.x; v.y *= inv * w.y; v.z *= inv * w.z; v.w *= inv * w.w;
      if (!gate_first) { v.x *= gk[j].x; v.y *= gk[j].y; v.z *= gk[j].z; v.w *= gk[j].w; }
      st4(dst + 4 * gi, v);
    }
  }
}

// A few segments of a long prompt leave most SMs without a block when a warp owns 8 columns:
// then a warp owns 2 and four times as many blocks share the work.
#ifndef NARROW_WC
#define NARROW_WC 2
#endif
static bool narrow_warps(int P, int heads, int S) {
  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return (long long)((P + 31) / 32) * heads * S < 2LL * sms;
}

template <typename AT, int NPL, int WC>
static int launch_ssd(SsdArgs a, int S, cudaStream_t stream) {
  constexpr int COLS = SCAN_WARPS * WC;
  const size_t smem = (size_t)2 * SCAN_CHUNK * (2 * a.N + COLS + 2) * sizeof(float);
  if (smem > 48 * 1024) return FT_ERR_SHAPE;
  a.vec = !(a.P % (WC % 4 == 0 ? 4 : 2)) && !(a.slot_stride % 4) && !((uintptr_t)a.state & 15);
  const dim3 grid((a.P + COLS - 1) / COLS, a.heads, S);
  cudaError_t e = launch_pdl(ssd_scan_kernel<AT, NPL, WC>, grid, dim3(SCAN_THREADS), smem, stream, a);
  return e == cudaSuccess ? FT_OK : (int)e;
}

template <typename AT, int NPL, int WC, int MODE = 0>
static int launch_delta(DeltaArgs a, int S, cudaStream_t stream) {
  constexpr int COLS = SCAN_WARPS * WC;
  const size_t smem = (size_t)2 * SCAN_CHUNK * ((MODE == 1 ? 3 : 2) * a.D + COLS + 2) * sizeof(float);
  if (smem > 96 * 1024) return FT_ERR_SHAPE;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(delta_scan_kernel<AT, NPL, WC, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  a.vec = !(a.P % (WC % 4 == 0 ? 4 : 2)) && !(a.slot_stride % 4) && !((uintptr_t)a.state & 15);
  const dim3 grid((a.P + COLS - 1) / COLS, a.heads, S);
  cudaError_t e = launch_pdl(delta_scan_kernel<AT, NPL, WC, MODE>, grid, dim3(SCAN_THREADS), smem, stream, a);
  return e == cudaSuccess ? FT_OK : (int)e;
}

template <int MODE>
static int dispatch_delta(DeltaArgs a, int S, int dtype, cudaStream_t stream) {
  int rc = FT_OK;
  const int D = a.D;
  const bool narrow = narrow_warps(a.P, a.heads, S);
  FT_DISPATCH(dtype, AT, {
    if (D <= 32) rc = narrow ? launch_delta<AT, 1, NARROW_WC, MODE>(a, S, stream) : launch_delta<AT, 1, 8, MODE>(a, S, stream);
    else if (D <= 64) rc = narrow ? launch_delta<AT, 2, NARROW_WC, MODE>(a, S, stream) : launch_delta<AT, 2, 8, MODE>(a, S, stream);
    else if (D <= 128) rc = narrow ? launch_delta<AT, 4, NARROW_WC, MODE>(a, S, stream) : launch_delta<AT, 4, 8, MODE>(a, S, stream);
    else rc = narrow ? launch_delta<AT, 8, NARROW_WC, MODE>(a, S, stream) : launch_delta<AT, 8, 8, MODE>(a, S, stream);
  });
  if (rc != FT_OK) return rc;
  FT_LAUNCH_CHECK();
  return FT_OK;
}

}  // namespace ft

using namespace ft;

extern "C" {

// Both kernels of the short convolution: outputs first, then the slots' new contents.
int ft_conv_silu(const void* x, long long ldx, void* out, long long ldo, const float* w, const float* bias,
                 float* state, long long slot_stride, const int* token_seg, const int* seg_slot,
                 const int* seg_q_start, int C, int taps, int T, int S, int dtype, int act, cudaStream_t stream) {
  if (T <= 0 || S <= 0) return FT_OK;
  if (C <= 0 || taps < 1) return FT_ERR_SHAPE;
  ConvArgs a{x, out, w, bias, state, token_seg, seg_slot, seg_q_start, ldx, ldo, slot_stride, C, taps, act};
  const int cb = (C + 127) / 128;
  if (taps > CONV_MAX_TAPS) {
    FT_DISPATCH(dtype, AT, launch_pdl(conv_silu_long_kernel<AT>, dim3(T, cb), dim3(128), 0, stream, a));
  } else {
    // many tokens: a thread walks 8 of them with its inputs in registers; few: a thread a token
    const bool many = T >= 1024;
    const dim3 rows(many ? (T + 7) / 8 : T);
    const bool pairs = dtype == FT_DTYPE_BF16 && !(C & 1) && !(ldx & 1) && !(ldo & 1) && !((uintptr_t)x & 3) &&
                       !((uintptr_t)out & 3);
    if (pairs) {
      const dim3 grid(rows.x, (C / 2 + 127) / 128);
      if (many) launch_pdl(conv_silu_kernel<__nv_bfloat16, 2, 8>, grid, dim3(128), 0, stream, a, T);
      else launch_pdl(conv_silu_kernel<__nv_bfloat16, 2, 1>, grid, dim3(128), 0, stream, a, T);
    } else if (many) {
      FT_DISPATCH(dtype, AT, launch_pdl(conv_silu_kernel<AT, 1, 8>, dim3(rows.x, cb), dim3(128), 0, stream, a, T));
    } else {
      FT_DISPATCH(dtype, AT, launch_pdl(conv_silu_kernel<AT, 1, 1>, dim3(rows.x, cb), dim3(128), 0, stream, a, T));
    }
  }
  FT_LAUNCH_CHECK();
  if (taps > 1) {
    FT_DISPATCH(dtype, AT, launch_pdl(conv_state_kernel<AT>, dim3(S, cb), dim3(128), 0, stream, a));
    FT_LAUNCH_CHECK();
  }
  return FT_OK;
}

int ft_ssd_scan(const void* xbc, long long ld, const void* dt, long long ld_dt, const float* dt_bias,
                const float* A_log, const float* D, float* state, long long slot_stride, float* y,
                const int* seg_slot, const int* seg_q_start, int heads, int P, int N, int G, int S,
                int dtype, cudaStream_t stream) {
  if (S <= 0) return FT_OK;
  if (heads <= 0 || P <= 0 || N <= 0 || N > 256 || G <= 0 || heads % G) return FT_ERR_SHAPE;
  SsdArgs a{xbc, dt, dt_bias, A_log, D, state, y, seg_slot, seg_q_start, ld, ld_dt, slot_stride, heads, P, N, G, 0};
  int rc = FT_OK;
  const bool narrow = narrow_warps(P, heads, S);
  FT_DISPATCH(dtype, AT, {
    if (N <= 32) rc = narrow ? launch_ssd<AT, 1, NARROW_WC>(a, S, stream) : launch_ssd<AT, 1, 8>(a, S, stream);
    else if (N <= 64) rc = narrow ? launch_ssd<AT, 2, NARROW_WC>(a, S, stream) : launch_ssd<AT, 2, 8>(a, S, stream);
    else if (N <= 128) rc = narrow ? launch_ssd<AT, 4, NARROW_WC>(a, S, stream) : launch_ssd<AT, 4, 8>(a, S, stream);
    else rc = narrow ? launch_ssd<AT, 8, NARROW_WC>(a, S, stream) : launch_ssd<AT, 8, 8>(a, S, stream);
  });
  if (rc != FT_OK) return rc;
  FT_LAUNCH_CHECK();
  return FT_OK;
}

int ft_delta_scan(const void* qkv, long long ld, const void* beta, const void* decay, long long ld_gate,
                  const float* dt_bias, const float* A_log, float* state, long long slot_stride, float* o,
                  const int* seg_slot, const int* seg_q_start, int heads, int P, int D, int G, float unit_eps,
                  float q_scale, int S, int dtype, cudaStream_t stream) {
  if (S <= 0) return FT_OK;
  if (heads <= 0 || P <= 0 || D <= 0 || D > 256 || G <= 0 || heads % G) return FT_ERR_SHAPE;
  DeltaArgs a{qkv, beta, decay, dt_bias, A_log, state, o, seg_slot, seg_q_start, ld, ld_gate, slot_stride,
              heads, P, D, G, unit_eps, q_scale, 0, nullptr, 0, nullptr, nullptr, 0};
  return dispatch_delta<0>(a, S, dtype, stream);
}

// The delta rule with a decay per key channel: `decay` is float32 [T, ld_decay] (channel n of head
// h at column h * D + n), dt_bias [heads * D].
int ft_channel_delta_scan(const void* qkv, long long ld, const void* beta, long long ld_gate, const float* decay,
                          long long ld_decay, const float* dt_bias, const float* A_log, float* state,
                          long long slot_stride, float* o, const int* seg_slot, const int* seg_q_start, int heads,
                          int P, int D, int G, float unit_eps, float q_scale, int S, int dtype,
                          cudaStream_t stream) {
  if (S <= 0) return FT_OK;
  if (heads <= 0 || P <= 0 || D <= 0 || D > 256 || G <= 0 || heads % G) return FT_ERR_SHAPE;
  DeltaArgs a{qkv, beta, nullptr, dt_bias, A_log, state, o, seg_slot, seg_q_start, ld, ld_gate, slot_stride,
              heads, P, D, G, unit_eps, q_scale, 0, decay, ld_decay, nullptr, nullptr, 0};
  return dispatch_delta<1>(a, S, dtype, stream);
}

// Retention: rows of `qkv` are q (heads * D) | k (heads * D) | v (heads * P); `decay` [heads] float32 holds
// each head's constant factor; cos_sin [positions, rot_dims] (rot_dims 0: nothing turns).
int ft_retention_scan(const void* qkv, long long ld, const float* decay, const float* cos_sin, int rot_dims,
                      const int* seg_pos0, float* state, long long slot_stride, float* o, const int* seg_slot,
                      const int* seg_q_start, int heads, int P, int D, float k_scale, int S, int dtype,
                      cudaStream_t stream) {
  if (S <= 0) return FT_OK;
  if (heads <= 0 || P <= 0 || D <= 0 || D > 256 || rot_dims < 0 || (rot_dims & 1) || rot_dims > D)
    return FT_ERR_SHAPE;
  DeltaArgs a{qkv, nullptr, nullptr, decay, nullptr, state, o, seg_slot, seg_q_start, ld, 0, slot_stride,
              heads, P, D, heads, 0.f, k_scale, 0, nullptr, 0, cos_sin, seg_pos0, cos_sin ? rot_dims : 0};
  return dispatch_delta<2>(a, S, dtype, stream);
}

int ft_gated_norm(const float* y, const void* z, long long ldz, const float* weight, int weight_len, void* out,
                  int T, int width, int groups, float eps, int gate_first, int gate_kind, int dtype,
                  cudaStream_t stream) {
  if (T <= 0) return FT_OK;
  if (width <= 0 || groups <= 0 || width % groups || weight_len <= 0) return FT_ERR_SHAPE;
  const long long items = (long long)T * groups;
  const int size = width / groups;
  const bool vec = !(size & 3) && !(weight_len & 3) && !(ldz & 3) && !((uintptr_t)y & 15) && !((uintptr_t)z & 15) &&
                   !((uintptr_t)weight & 15) && !((uintptr_t)out & 15);
  if (vec && size <= 16 * 32) {
    FT_DISPATCH(dtype, AT, launch_pdl(gated_norm_vec_kernel<AT, 32, 4>, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, stream,
                                      y, (const AT*)z, ldz, weight, weight_len, (AT*)out, T, width, groups, eps,
                                      gate_first, gate_kind));
    FT_LAUNCH_CHECK();
    return FT_OK;
  }
  if (vec && size <= 16 * 128) {
    FT_DISPATCH(dtype, AT, launch_pdl(gated_norm_vec_kernel<AT, 128, 4>, dim3((unsigned)items), dim3(128), 0, stream, y,
                                      (const AT*)z, ldz, weight, weight_len, (AT*)out, T, width, groups, eps,
                                      gate_first, gate_kind));
    FT_LAUNCH_CHECK();
    return FT_OK;
  }
  if (vec && size <= 64 * 128) {
    FT_DISPATCH(dtype, AT, launch_pdl(gated_norm_vec_kernel<AT, 128, 16>, dim3((unsigned)items), dim3(128), 0, stream, y,
                                      (const AT*)z, ldz, weight, weight_len, (AT*)out, T, width, groups, eps,
                                      gate_first, gate_kind));
    FT_LAUNCH_CHECK();
    return FT_OK;
  }
  const unsigned blocks = (unsigned)((items + 3) / 4);
  FT_DISPATCH(dtype, AT, launch_pdl(gated_norm_kernel<AT>, dim3(blocks), dim3(128), 0, stream, y, (const AT*)z, ldz,
                                    weight, weight_len, (AT*)out, T, width, groups, eps, gate_first, gate_kind));
  FT_LAUNCH_CHECK();
  return FT_OK;
}

}  // extern "C"
