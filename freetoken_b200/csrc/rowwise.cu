// Row-wise kernels of mixers that keep ONE tensor per token in the cache (keys
// that are also the values, or a latent vector), of plain two-matrix
// feed-forwards, and of heads and embeddings with a norm or a cap of their own.
//
// All arithmetic is float32 whatever the storage type; a block (or a thread)
// owns one token, so a token's result does not depend on what else is in the
// launch.
//
//   embed_norm      r[t,:] = rms(E[id_t,:]) * g          (gather + RMS norm in one pass)
//   embed_pair      r[t,:] = E[id_t,:] * scale + B[hash(id_{t-1}, id_t),:]
//   key_store       q_out[t,h,:] = q[t,h,:] * (1 + coef * ln(floor((p_t + 1) / every) + 1))
//                   k[t,g,:] -> (optionally rms(k) * w, per key head) -> page of p_t
//   gate_heads      o[t,h,:] *= sigmoid(z[t,h])
//   activation      y = f(x): relu(x)^2, tanh-GELU, SiLU
//   softcap         y = cap * tanh(y / cap)
#include "common.cuh"

namespace ft {

// ------------------------------------------------------------- embed + norm
// 4 consecutive elements as float32
__device__ __forceinline__ float4 load4f(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4f(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}

constexpr int EMBED_THREADS = 256;
constexpr int EMBED_KEEP = 4;      // groups of 4 elements a thread keeps between the two passes

// VEC: rows of up to 4 * EMBED_THREADS * EMBED_KEEP elements, a multiple of 4, 16-byte aligned:
// the row is read once and stays in registers between the sum of squares and the scaling.
template <typename WT, bool VEC>
__global__ void __launch_bounds__(EMBED_THREADS)
embed_norm_kernel(const int* __restrict__ ids, const WT* __restrict__ table,
                  const float* __restrict__ weight, float* __restrict__ residual, int H, int vocab,
                  float eps) {
  __shared__ float scratch[33];
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) id = 0;  // validated on the host; never index outside the table
  const WT* row = table + (size_t)id * H;
  float* out = residual + (size_t)t * H;
  float ss = 0.f;
  if (VEC) {
    float4 keep[EMBED_KEEP];
    const int groups = H >> 2;
#pragma unroll
    for (int j = 0; j < EMBED_KEEP; ++j) {
      const int gi = threadIdx.x + j * EMBED_THREADS;
      if (gi < groups) {
        const float4 v = load4f(row + 4 * gi);
        keep[j] = v;
        ss += v.x * v.x;
        ss += v.y * v.y;
        ss += v.z * v.z;
        ss += v.w * v.w;
      }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
    for (int j = 0; j < EMBED_KEEP; ++j) {
      const int gi = threadIdx.x + j * EMBED_THREADS;
      if (gi < groups) {
        const float4 w = load4f(weight + 4 * gi);
        const float4 v = keep[j];
        *reinterpret_cast<float4*>(out + 4 * gi) = make_float4(v.x * inv * w.x, v.y * inv * w.y, v.z * inv * w.z,
                                                               v.w * inv * w.w);
      }
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      const float v = to_float(row[i]);
      ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[i] = to_float(row[i]) * inv * weight[i];
  }
}

// ---------------------------------------------------------------- key store
struct KeyStoreArgs {
  const void* src;        // [T, ld]: a projection's rows; queries at q_off, keys at k_off
  void* q_out;            // [T, nq*dq] or nullptr (queries are left where they are)
  void* pages;            // [pages, nkv, P, dk] or nullptr (a stop that reads another stop's cache)
  const float* k_weight;  // [dk] or nullptr: RMS norm of every key head's row, times this
  const int* token_pos;   // [T]
  const int* token_seg;   // [T]
  const int* block_table; // [S, table_width]
  long long ld, page_stride;
  int q_off, k_off, nq, dq, nkv, dk, P, table_width, every;
  float coef, eps;
};

// 8 consecutive bfloat16 values as float32, and back
__device__ __forceinline__ void unpack8(const uint4& raw, float (&v)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  return raw;
}

// A block takes `tokens_per_block` tokens (1 when there are queries to scale: all its threads
// share them; more when only keys are stored); a warp takes one (token, key head) row at a time.
// VEC (bfloat16, everything a multiple of 8 elements and 16-byte aligned): 16-byte pieces.
template <typename AT, bool VEC>
__global__ void __launch_bounds__(128) key_store_kernel(KeyStoreArgs a, int T, int tokens_per_block) {
  pdl_wait();
  const int t0 = blockIdx.x * tokens_per_block;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  if (a.q_out) {
    // the temperature is a function of the position alone, in float32
    const int t = t0;
    const AT* q = (const AT*)a.src + (size_t)t * a.ld + a.q_off;
    const int pos = a.token_pos[t];
    float temp = 1.f;
    if (a.coef != 0.f) temp = 1.f + a.coef * logf((float)((pos + 1) / a.every) + 1.f);
    AT* qo = (AT*)a.q_out + (size_t)t * a.nq * a.dq;
    const int n = a.nq * a.dq;
    if (VEC) {
      for (int c = threadIdx.x; c < (n >> 3); c += blockDim.x) {
        float v[8];
        unpack8(*reinterpret_cast<const uint4*>(q + 8 * c), v);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] *= temp;
        *reinterpret_cast<uint4*>(qo + 8 * c) = pack8(v);
      }
    } else {
      for (int i = threadIdx.x; i < n; i += blockDim.x) qo[i] = from_float<AT>(to_float(q[i]) * temp);
    }
  }
  if (!a.pages) return;
  for (int r = warp; r < tokens_per_block * a.nkv; r += nwarps) {
    const int t = t0 + r / a.nkv, g = r % a.nkv;
    if (t >= T) break;
    const int pos = a.token_pos[t];
    const int page = a.block_table[(size_t)a.token_seg[t] * a.table_width + pos / a.P];
    const AT* k = (const AT*)a.src + (size_t)t * a.ld + a.k_off + (size_t)g * a.dk;
    AT* kd = (AT*)a.pages + (size_t)page * a.page_stride + ((size_t)g * a.P + pos % a.P) * a.dk;
    if (VEC) {
      const int chunks = a.dk >> 3;
      float first[8];                       // the lane's first piece stays in registers
      float ss = 0.f;
      for (int c = lane; c < chunks; c += 32) {
        float v[8];
        unpack8(*reinterpret_cast<const uint4*>(k + 8 * c), v);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          ss += v[i] * v[i];
          if (c == lane) first[i] = v[i];
        }
      }
      float inv = 1.f;
      if (a.k_weight) inv = 1.0f / sqrtf(warp_sum(ss) / (float)a.dk + a.eps);
      for (int c = lane; c < chunks; c += 32) {
        float v[8];
        if (c == lane) {
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = first[i];
        } else {
          unpack8(*reinterpret_cast<const uint4*>(k + 8 * c), v);
        }
        if (a.k_weight) {
          const float4 w0 = *reinterpret_cast<const float4*>(a.k_weight + 8 * c);
          const float4 w1 = *reinterpret_cast<const float4*>(a.k_weight + 8 * c + 4);
          v[0] *= inv * w0.x; v[1] *= inv * w0.y; v[2] *= inv * w0.z; v[3] *= inv * w0.w;
          v[4] *= inv * w1.x; v[5] *= inv * w1.y; v[6] *= inv * w1.z; v[7] *= inv * w1.w;
        }
        *reinterpret_cast<uint4*>(kd + 8 * c) = pack8(v);
      }
    } else if (a.k_weight) {
      float ss = 0.f;
      for (int i = lane; i < a.dk; i += 32) {
        const float v = to_float(k[i]);
        ss += v * v;
      }
      ss = warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss / (float)a.dk + a.eps);
      for (int i = lane; i < a.dk; i += 32) kd[i] = from_float<AT>(to_float(k[i]) * inv * a.k_weight[i]);
    } else {
      for (int i = lane; i < a.dk; i += 32) kd[i] = k[i];
    }
  }
}

// ------------------------------------------------------------------- gates
// o[t, h, 0..d) *= sigmoid(z[t*ldz + h]).  A thread owns PIECE consecutive elements of one head
// (8 bfloat16 values as one 16-byte piece when d allows it), so the gate is evaluated once a piece.
template <typename AT, int PIECE>
__global__ void __launch_bounds__(256)
gate_heads_kernel(AT* __restrict__ o, const AT* __restrict__ z, long long ldz, int heads, int d, long long pieces) {
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= pieces) return;
  const long long th = i / (d / PIECE);
  const long long t = th / heads;
  const int h = (int)(th - t * heads);
  const float zz = to_float(z[t * ldz + h]);
  const float g = 1.f / (1.f + expf(-zz));
  if (PIECE == 8) {
    uint4* p = reinterpret_cast<uint4*>(o) + i;
    uint4 raw = *p;
    __nv_bfloat162* v = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(v[j]);
      v[j] = __floats2bfloat162_rn(f.x * g, f.y * g);
    }
    *p = raw;
  } else {
    o[i] = from_float<AT>(to_float(o[i]) * g);
  }
}

// -------------------------------------------------------------- activation
__device__ __forceinline__ float act_apply(float x, int kind) {
  switch (kind) {
    case 0: { const float r = fmaxf(x, 0.f); return r * r; }                     // relu squared
    case 1: return 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));  // tanh-GELU
    default: return x / (1.f + expf(-x));                                         // SiLU
  }
}

template <typename AT>
__global__ void __launch_bounds__(256) activation_kernel(AT* __restrict__ x, long long n, int kind) {
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] = from_float<AT>(act_apply(to_float(x[i]), kind));
}

// 8 bfloat16 values a thread
__global__ void __launch_bounds__(256) activation_bf16x8_kernel(uint4* __restrict__ x, long long n8, int kind) {
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  uint4 raw = x[i];
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 v = __bfloat1622float2(p[j]);
    p[j] = __floats2bfloat162_rn(act_apply(v.x, kind), act_apply(v.y, kind));
  }
  x[i] = raw;
}

// ------------------------------------------------------------------ softcap
__global__ void __launch_bounds__(256) softcap_kernel(float* __restrict__ x, long long n, float cap) {
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] = cap * tanhf(x[i] / cap);
}

// ------------------------------------------------- a branch's own norm, then the residual
// z = sum_j s_j * branch[t, j, :] (float32; s_j = 1 without scales); the residual takes
// mult * rms(z) * (w [+1]).  With a second weight the new residual row is normed once more
// in the same pass and leaves as the next sublayer's input.  A block owns a token; z, then the
// new residual row, stay in shared memory between the passes.
__device__ __forceinline__ void store4f(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4f(__nv_bfloat16* p, float4 v) {
  uint2 raw;
  *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v.x, v.y);
  *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = raw;
}

constexpr int NORM_ADD_KEEP = 8;   // groups of 4 elements a thread keeps between the passes

// VEC: rows of up to 4 * 256 * NORM_ADD_KEEP elements, a multiple of 4, every row 16-byte (bfloat16: 8-byte)
// aligned: each row is read once, in 16-byte pieces, and stays in registers between the passes.
template <typename AT, bool VEC>
__global__ void __launch_bounds__(256)
norm_add_kernel(const AT* __restrict__ branch, int k, const float* __restrict__ part_scale,
                const float* __restrict__ weight, int plus_one, float eps, float mult,
                float* __restrict__ residual, const float* __restrict__ next_weight, int next_plus_one,
                float next_eps, AT* __restrict__ next_out, int H) {
  extern __shared__ float row[];
  __shared__ float scratch[33];
  pdl_wait();
  const int t = blockIdx.x;
  const AT* b = branch + (size_t)t * k * H;
  float* r = residual + (size_t)t * H;
  const float one = plus_one ? 1.f : 0.f;
  const float one2 = next_plus_one ? 1.f : 0.f;
  float ss = 0.f, ss2 = 0.f;
  if constexpr (VEC) {
    float4 keep[NORM_ADD_KEEP];
    const int groups = H >> 2;
#pragma unroll
    for (int j = 0; j < NORM_ADD_KEEP; ++j) {
      const int gi = threadIdx.x + j * 256;
      if (gi < groups) {
        float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int q = 0; q < k; ++q) {
          const float4 v = load4f(b + (size_t)q * H + 4 * gi);
          if (part_scale) {
            const float s = part_scale[q];
            z.x = fmaf(s, v.x, z.x); z.y = fmaf(s, v.y, z.y); z.z = fmaf(s, v.z, z.z); z.w = fmaf(s, v.w, z.w);
          } else {
            z.x += v.x; z.y += v.y; z.z += v.z; z.w += v.w;
          }
        }
        keep[j] = z;
        ss = fmaf(z.x, z.x, ss); ss = fmaf(z.y, z.y, ss); ss = fmaf(z.z, z.z, ss); ss = fmaf(z.w, z.w, ss);
      }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
    for (int j = 0; j < NORM_ADD_KEEP; ++j) {
      const int gi = threadIdx.x + j * 256;
      if (gi < groups) {
        const float4 w = load4f(weight + 4 * gi), x0 = load4f(r + 4 * gi), z = keep[j];
        const float4 x = make_float4(x0.x + mult * (z.x * inv * (w.x + one)), x0.y + mult * (z.y * inv * (w.y + one)),
                                     x0.z + mult * (z.z * inv * (w.z + one)), x0.w + mult * (z.w * inv * (w.w + one)));
        store4f(r + 4 * gi, x);
        keep[j] = x;
        ss2 = fmaf(x.x, x.x, ss2); ss2 = fmaf(x.y, x.y, ss2); ss2 = fmaf(x.z, x.z, ss2); ss2 = fmaf(x.w, x.w, ss2);
      }
    }
    if (!next_weight) return;
    ss2 = block_sum(ss2, scratch);
    const float inv2 = 1.0f / sqrtf(ss2 / (float)H + next_eps);
    AT* o = next_out + (size_t)t * H;
#pragma unroll
    for (int j = 0; j < NORM_ADD_KEEP; ++j) {
      const int gi = threadIdx.x + j * 256;
      if (gi < groups) {
        const float4 w = load4f(next_weight + 4 * gi), x = keep[j];
        store4f(o + 4 * gi, make_float4(x.x * inv2 * (w.x + one2), x.y * inv2 * (w.y + one2), x.z * inv2 * (w.z + one2),
                                        x.w * inv2 * (w.w + one2)));
      }
    }
    return;
  } else {
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float z = 0.f;
    for (int j = 0; j < k; ++j) {
      const float v = to_float(b[(size_t)j * H + i]);
      z = part_scale ? fmaf(part_scale[j], v, z) : z + v;
    }
    row[i] = z;
    ss = fmaf(z, z, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float x = r[i] + mult * (row[i] * inv * (weight[i] + one));
    r[i] = x;
    row[i] = x;
    ss2 = fmaf(x, x, ss2);
  }
  if (!next_weight) return;
  ss2 = block_sum(ss2, scratch);
  const float inv2 = 1.0f / sqrtf(ss2 / (float)H + next_eps);
  AT* o = next_out + (size_t)t * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_float<AT>(row[i] * inv2 * (next_weight[i] + one2));
  }
}

// out[t, :] = sum_j s_j * parts[t, j, :]   (float32 sum, ascending j)
template <typename AT>
__global__ void __launch_bounds__(256)
scaled_sum_kernel(const AT* __restrict__ parts, const float* __restrict__ scale, AT* __restrict__ out, int k,
                  long long n, int H) {
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long long t = i / H;
  const int c = (int)(i - t * H);
  float z = 0.f;
  for (int j = 0; j < k; ++j) z = fmaf(scale[j], to_float(parts[((size_t)t * k + j) * H + c]), z);
  out[i] = from_float<AT>(z);
}

// x[t, c] += bias[c]; rows may lie further apart than their width
template <typename AT>
__global__ void __launch_bounds__(256)
bias_add_kernel(AT* __restrict__ x, long long ld, const float* __restrict__ bias, long long n, int width) {
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long long t = i / width;
  const int c = (int)(i - t * width);
  AT* p = x + t * ld + c;
  *p = from_float<AT>(to_float(*p) + bias[c]);
}

// mid[t, i] = f(gu[t, i]) * gu[t, I + i]: the gate and up halves of one merged projection
// kind 3: the clamped pair  g = min(gate, limit), u = clamp(up, -limit, limit),  g sigmoid(alpha g) (u + 1)
template <typename AT>
__global__ void __launch_bounds__(256)
glu_rows_kernel(const AT* __restrict__ gu, AT* __restrict__ mid, long long n, int I, int kind, float alpha,
                float limit) {
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long long t = i / I;
  const int c = (int)(i - t * I);
  const AT* row = gu + (size_t)t * 2 * I;
  const float gate = to_float(row[c]), up = to_float(row[I + c]);
  float v;
  if (kind == 3) {
    const float g = fminf(gate, limit), u = fminf(fmaxf(up, -limit), limit);
    v = g / (1.f + expf(-alpha * g)) * (u + 1.f);
  } else {
    v = act_apply(gate, kind) * up;
  }
  mid[i] = from_float<AT>(v);
}

// ------------------------------------------------- several residual streams (hyper-connections)
// A token has S residual streams x_0 .. x_{S-1} (float32, [T, S, H]).  One launch, per token:
//   1. the pending branch output y (the sum of its k partial rows, ascending) joins the streams:
//        x_t <- sum_s mix[s, t] x_s + out[t] y          (all t from the old x; skipped without a branch)
//   2. the next sublayer's input  u = sum_s read[s] x_s   (read == nullptr: the plain sum)
//   3. layer norm (mean, then the mean of the squared deviations, eps inside the root, weight and
//      bias) or RMS norm (no bias) of u into `normed` in the activation type.
// One block per token; u is kept in shared memory between the passes; every sum has a fixed order.
constexpr int HYPER_MAX_STREAMS = 8;
template <typename AT>
__global__ void __launch_bounds__(256)
hyper_norm_kernel(float* __restrict__ streams, const AT* __restrict__ branch, int k, const float* __restrict__ mix,
                  const float* __restrict__ out_w, const float* __restrict__ read, const float* __restrict__ weight,
                  const float* __restrict__ bias, float eps, int center, AT* __restrict__ normed, int S, int H) {
  extern __shared__ float u_row[];
  __shared__ float scratch[33];
  __shared__ float s_mix[HYPER_MAX_STREAMS * HYPER_MAX_STREAMS], s_out[HYPER_MAX_STREAMS], s_read[HYPER_MAX_STREAMS];
  pdl_wait();
  const int t = blockIdx.x;
  if (threadIdx.x < S * S) s_mix[threadIdx.x] = branch ? mix[threadIdx.x] : 0.f;
  if (threadIdx.x < S) {
    s_out[threadIdx.x] = branch ? out_w[threadIdx.x] : 0.f;
    s_read[threadIdx.x] = read ? read[threadIdx.x] : 1.f;
  }
  __syncthreads();
  float* x = streams + (size_t)t * S * H;
  const AT* y_rows = branch ? branch + (size_t)t * k * H : nullptr;
  float sum = 0.f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float xs[HYPER_MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < HYPER_MAX_STREAMS; ++s) xs[s] = s < S ? x[(size_t)s * H + c] : 0.f;
    if (branch) {
      float y = 0.f;
      for (int j = 0; j < k; ++j) y += to_float(y_rows[(size_t)j * H + c]);
      float nx[HYPER_MAX_STREAMS];
#pragma unroll
      for (int r = 0; r < HYPER_MAX_STREAMS; ++r) {
        float v = 0.f;
        if (r < S) {
#pragma unroll
          for (int s = 0; s < HYPER_MAX_STREAMS; ++s)
            if (s < S) v = fmaf(s_mix[s * S + r], xs[s], v);
          v = fmaf(s_out[r], y, v);
          x[(size_t)r * H + c] = v;
        }
        nx[r] = v;
      }
#pragma unroll
      for (int s = 0; s < HYPER_MAX_STREAMS; ++s) xs[s] = nx[s];
    }
    float u = 0.f;
#pragma unroll
    for (int s = 0; s < HYPER_MAX_STREAMS; ++s)
      if (s < S) u = fmaf(s_read[s], xs[s], u);
    u_row[c] = u;
    sum += u;
  }
  if (!normed) return;
  float mean = 0.f;
  if (center) mean = block_sum(sum, scratch) / (float)H;
  float sq = 0.f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    const float d = u_row[c] - mean;
    sq = fmaf(d, d, sq);
  }
  const float inv = 1.f / sqrtf(block_sum(sq, scratch) / (float)H + eps);
  AT* dst = normed + (size_t)t * H;
  for (int c = threadIdx.x; c < H; c += blockDim.x)
    dst[c] = from_float<AT>((u_row[c] - mean) * inv * weight[c] + (bias ? bias[c] : 0.f));
}

// The same launch for rows of a multiple of 4 values with 16-byte aligned rows, S known at compile time:
// a thread owns up to KEEP groups of 4 consecutive values; it first fetches all its pieces of every
// stream and of the branch (all loads in flight together), then joins, reads and keeps u in registers
// between the passes.  The sums run in the order of the generic kernel.
template <typename AT, int S, int KEEP>
__global__ void __launch_bounds__(256)
hyper_norm_vec_kernel(float* __restrict__ streams, const AT* __restrict__ branch, int k, const float* __restrict__ mix,
                      const float* __restrict__ out_w, const float* __restrict__ read,
                      const float* __restrict__ weight, const float* __restrict__ bias, float eps, int center,
                      AT* __restrict__ normed, int H) {
  __shared__ float scratch[33];
  pdl_wait();
  const int t = blockIdx.x, groups = H >> 2;
  float m[S * S], ow[S], rd[S];
#pragma unroll
  for (int i = 0; i < S * S; ++i) m[i] = branch ? mix[i] : 0.f;
#pragma unroll
  for (int i = 0; i < S; ++i) {
    ow[i] = branch ? out_w[i] : 0.f;
    rd[i] = read ? read[i] : 1.f;
  }
  float* x = streams + (size_t)t * S * H;
  const AT* y_rows = branch ? branch + (size_t)t * k * H : nullptr;
  float4 xs[KEEP][S], y[KEEP];
#pragma unroll
  for (int j = 0; j < KEEP; ++j) {
    const int gi = threadIdx.x + j * 256;
    y[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (gi < groups) {
#pragma unroll
      for (int s_ = 0; s_ < S; ++s_) xs[j][s_] = load4f(x + (size_t)s_ * H + 4 * gi);
      if (branch) {
        for (int q = 0; q < k; ++q) {
          const float4 v = load4f(y_rows + (size_t)q * H + 4 * gi);
          y[j].x += v.x; y[j].y += v.y; y[j].z += v.z; y[j].w += v.w;
        }
      }
    }
  }
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < KEEP; ++j) {
    const int gi = threadIdx.x + j * 256;
    if (gi < groups) {
      float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
      if (branch) {
#pragma unroll
        for (int r = 0; r < S; ++r) {
          float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int s_ = 0; s_ < S; ++s_) {
            const float c = m[s_ * S + r];
            v.x = fmaf(c, xs[j][s_].x, v.x); v.y = fmaf(c, xs[j][s_].y, v.y);
            v.z = fmaf(c, xs[j][s_].z, v.z); v.w = fmaf(c, xs[j][s_].w, v.w);
          }
          v.x = fmaf(ow[r], y[j].x, v.x); v.y = fmaf(ow[r], y[j].y, v.y);
          v.z = fmaf(ow[r], y[j].z, v.z); v.w = fmaf(ow[r], y[j].w, v.w);
          store4f(x + (size_t)r * H + 4 * gi, v);
          u.x = fmaf(rd[r], v.x, u.x); u.y = fmaf(rd[r], v.y, u.y); u.z = fmaf(rd[r], v.z, u.z); u.w = fmaf(rd[r], v.w, u.w);
        }
      } else {
#pragma unroll
        for (int s_ = 0; s_ < S; ++s_) {
          u.x = fmaf(rd[s_], xs[j][s_].x, u.x); u.y = fmaf(rd[s_], xs[j][s_].y, u.y);
          u.z = fmaf(rd[s_], xs[j][s_].z, u.z); u.w = fmaf(rd[s_], xs[j][s_].w, u.w);
        }
      }
      y[j] = u;
      sum += u.x; sum += u.y; sum += u.z; sum += u.w;
    }
  }
  if (!normed) return;
  float mean = 0.f;
  if (center) mean = block_sum(sum, scratch) / (float)H;
  float sq = 0.f;
#pragma unroll
  for (int j = 0; j < KEEP; ++j) {
    if ((int)threadIdx.x + j * 256 < groups) {
      float4& u = y[j];
      u.x -= mean; u.y -= mean; u.z -= mean; u.w -= mean;
      sq = fmaf(u.x, u.x, sq); sq = fmaf(u.y, u.y, sq); sq = fmaf(u.z, u.z, sq); sq = fmaf(u.w, u.w, sq);
    }
  }
  const float inv = 1.f / sqrtf(block_sum(sq, scratch) / (float)H + eps);
  AT* dst = normed + (size_t)t * H;
#pragma unroll
  for (int j = 0; j < KEEP; ++j) {
    const int gi = threadIdx.x + j * 256;
    if (gi < groups) {
      const float4 w = load4f(weight + 4 * gi);
      const float4 b = bias ? load4f(bias + 4 * gi) : make_float4(0.f, 0.f, 0.f, 0.f);
      const float4 u = y[j];
      store4f(dst + 4 * gi, make_float4(u.x * inv * w.x + b.x, u.y * inv * w.y + b.y, u.z * inv * w.z + b.z,
                                        u.w * inv * w.w + b.w));
    }
  }
}

template <typename AT, int S>
static cudaError_t launch_hyper_vec(cudaStream_t stream, int T, int H, float* streams, const AT* branch, int k,
                                    const float* mix, const float* out_w, const float* read, const float* weight,
                                    const float* bias, float eps, int center, AT* normed) {
  if (H <= 2048)
    return launch_pdl(hyper_norm_vec_kernel<AT, S, 2>, dim3(T), dim3(256), 0, stream, streams, branch, k, mix, out_w,
                      read, weight, bias, eps, center, normed, H);
  if (H <= 4096)
    return launch_pdl(hyper_norm_vec_kernel<AT, S, 4>, dim3(T), dim3(256), 0, stream, streams, branch, k, mix, out_w,
                      read, weight, bias, eps, center, normed, H);
  return launch_pdl(hyper_norm_vec_kernel<AT, S, 8>, dim3(T), dim3(256), 0, stream, streams, branch, k, mix, out_w, read,
                    weight, bias, eps, center, normed, H);
}

// Rows of a column range of a wider matrix, RMS-normed and multiplied by a weight:
// out[t, :] = x[t, :] / sqrt(mean(x[t, :]^2) + eps) * w.   One block per row.
template <typename AT>
__global__ void __launch_bounds__(128)
rms_rows_kernel(const AT* __restrict__ x, long long ldx, const float* __restrict__ w, AT* __restrict__ out,
                long long ldo, int n, float eps) {
  __shared__ float scratch[33];
  pdl_wait();
  const AT* row = x + (size_t)blockIdx.x * ldx;
  float sq = 0.f;
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    const float v = to_float(row[c]);
    sq = fmaf(v, v, sq);
  }
  const float inv = 1.f / sqrtf(block_sum(sq, scratch) / (float)n + eps);
  AT* dst = out + (size_t)blockIdx.x * ldo;
  for (int c = threadIdx.x; c < n; c += blockDim.x) dst[c] = from_float<AT>(to_float(row[c]) * inv * w[c]);
}

// What latent attention with a rotated key part does between its projections and its attention.
// Per token: the latent (rank values of the down projection's row) is RMS-normed, times its weight,
// and stored in the token's place of the page; the rot values behind it are turned by the token's
// position (dimension 2i with 2i + 1, or i with i + rot/2) and stored behind the latent: a cached
// row is [latent | rotated key part].  The rotated part of every head's query (the last rot of its
// dq + rot values) is turned the same way and written behind the first rank values of the head's
// row of q_abs ([T, heads, rank + rot]), whose first rank values another product fills.
struct LatentStoreArgs {
  const void* down;        // [T, ld_down]: latent at column 0, the key part to rotate at column rank
  const void* q;           // [T, ld_q]: head h at column h * (dq + rot)
  void* q_abs;             // [T, heads, rank + rot]
  void* pages;             // [pages, 1, P, rank + rot] or nullptr
  const float* weight;     // [rank]
  const float* cos_sin;    // [positions, rot]: cos | sin
  const int* token_pos;
  const int* token_seg;
  const int* block_table;  // [segments, table_width]
  long long ld_down, ld_q, page_stride;
  int heads, dq, rank, rot, P, table_width, interleaved;
  float eps;
};

template <typename AT>
__global__ void __launch_bounds__(128) latent_store_kernel(LatentStoreArgs a) {
  __shared__ float scratch[33];
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = a.token_pos[t];
  const int half = a.rot >> 1;
  const float* cs = a.cos_sin + (size_t)pos * a.rot;
  auto turn = [&](const AT* src, AT* dst, int i) {       // pair i of a rotated part
    const int ia = a.interleaved ? 2 * i : i, ib = a.interleaved ? 2 * i + 1 : i + half;
    const float u = to_float(src[ia]), v = to_float(src[ib]);
    const float c = cs[i], s = cs[half + i];
    dst[ia] = from_float<AT>(u * c - v * s);
    dst[ib] = from_float<AT>(v * c + u * s);
  };
  const int width = a.rank + a.rot;
  // queries: the rotated part of every head
  const AT* q = (const AT*)a.q + (size_t)t * a.ld_q;
  AT* qa = (AT*)a.q_abs + (size_t)t * a.heads * width;
  for (int i = threadIdx.x; i < a.heads * half; i += blockDim.x) {
    const int h = i / half, p = i - h * half;
    turn(q + (size_t)h * (a.dq + a.rot) + a.dq, qa + (size_t)h * width + a.rank, p);
  }
  if (!a.pages) return;
  const AT* down = (const AT*)a.down + (size_t)t * a.ld_down;
  const int page = a.block_table[(size_t)a.token_seg[t] * a.table_width + pos / a.P];
  AT* dst = (AT*)a.pages + (size_t)page * a.page_stride + (size_t)(pos % a.P) * width;
  float sq = 0.f;
  for (int c = threadIdx.x; c < a.rank; c += blockDim.x) {
    const float v = to_float(down[c]);
    sq = fmaf(v, v, sq);
  }
  const float inv = 1.f / sqrtf(block_sum(sq, scratch) / (float)a.rank + a.eps);
  for (int c = threadIdx.x; c < a.rank; c += blockDim.x)
    dst[c] = from_float<AT>(to_float(down[c]) * inv * a.weight[c]);
  for (int i = threadIdx.x; i < half; i += blockDim.x) turn(down + a.rank, dst + a.rank, i);
}


// ------------------------------------------------- embedding with a second, hashed table
// r[t,:] = E[id_t,:] * scale + B[row_t,:] where row_t = (prev_t * mul_prev + id_t * mul_cur) mod
// buckets and prev_t is the token before t in its sequence; a sequence's first token takes row
// `buckets`, the table's last.  The token before a portion's first token is what the request's
// slot carries (one int32 a slot); the block of a portion's first token reads it and then leaves
// the portion's last token there, so nobody else touches the slot in this launch.  The sum is
// float32 and is written to every one of `copies` residual streams.
struct EmbedPairArgs {
  const int* ids;          // [T]
  const int* token_pos;    // [T]
  const int* token_seg;    // [T]
  const int* seg_slot;     // [S]
  const int* seg_q_start;  // [S + 1]
  const void* table;       // [vocab, H]
  const void* pair_table;  // [buckets + 1, H], or nullptr: no second table
  int* last_token;         // slot s: last_token[s * slot_stride]
  float* residual;         // [T, copies, H]
  long long slot_stride;
  long long mul_prev, mul_cur;
  int buckets, H, vocab, copies;
  float scale;
};

template <typename WT>
__global__ void __launch_bounds__(256) embed_pair_kernel(EmbedPairArgs a) {
  pdl_wait();
  const int t = blockIdx.x;
  int id = a.ids[t];
  if (id < 0 || id >= a.vocab) id = 0;  // validated on the host; never index outside the table
  const WT* row = (const WT*)a.table + (size_t)id * a.H;
  const WT* pair = nullptr;
  if (a.pair_table) {
    const int seg = a.token_seg[t];
    const int q0 = a.seg_q_start[seg];
    long long r = a.buckets;
    if (a.token_pos[t] > 0) {
      int prev = t > q0 ? a.ids[t - 1] : a.last_token[(size_t)a.seg_slot[seg] * a.slot_stride];
      if (prev < 0 || prev >= a.vocab) prev = 0;
      r = ((long long)prev * a.mul_prev + (long long)id * a.mul_cur) % a.buckets;
      if (r < 0) r += a.buckets;
    }
    pair = (const WT*)a.pair_table + (size_t)r * a.H;
    if (t == q0) {
      // all threads have read the slot (or will not): the slot's new content is this portion's last token
      __syncthreads();
      if (threadIdx.x == 0) a.last_token[(size_t)a.seg_slot[seg] * a.slot_stride] = a.ids[a.seg_q_start[seg + 1] - 1];
    }
  }
  float* out = a.residual + (size_t)t * a.H * a.copies;
  // four elements a step where the rows allow it (8-byte loads of bfloat16, 16-byte stores)
  if ((a.H & 3) == 0 && (((uintptr_t)a.table | (uintptr_t)a.pair_table | (uintptr_t)a.residual) & 15) == 0 &&
      (a.H * sizeof(WT)) % 16 == 0) {
    for (int i = threadIdx.x; i < (a.H >> 2); i += blockDim.x) {
      float4 v = load4f(row + 4 * i);
      v.x *= a.scale; v.y *= a.scale; v.z *= a.scale; v.w *= a.scale;
      if (pair) {
        const float4 b = load4f(pair + 4 * i);
        v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
      }
      for (int c = 0; c < a.copies; ++c) *reinterpret_cast<float4*>(out + (size_t)c * a.H + 4 * i) = v;
    }
    return;
  }
  for (int i = threadIdx.x; i < a.H; i += blockDim.x) {
    float v = to_float(row[i]) * a.scale;
    if (pair) v += to_float(pair[i]);
    for (int c = 0; c < a.copies; ++c) out[(size_t)c * a.H + i] = v;
  }
}

// o[t, i] *= sigmoid(z[t, i]): a gate per value, 16-byte pieces of eight bfloat16 values (the sigmoid from the
// fast exponential and division: float32 arithmetic whose error lies far below the bfloat16 result's rounding)
__global__ void __launch_bounds__(256)
gate_values_bf16x8_kernel(__nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ z, long long ldz, int n8,
                          long long pieces) {
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= pieces) return;
  const long long t = i / n8;
  const int c = (int)(i - t * n8);
  uint4* p = reinterpret_cast<uint4*>(o) + i;
  uint4 raw = *p;
  const uint4 zr = *reinterpret_cast<const uint4*>(z + t * ldz + 8 * c);
  __nv_bfloat162* v = reinterpret_cast<__nv_bfloat162*>(&raw);
  const __nv_bfloat162* g = reinterpret_cast<const __nv_bfloat162*>(&zr);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __bfloat1622float2(v[j]), zz = __bfloat1622float2(g[j]);
    v[j] = __floats2bfloat162_rn(__fdividef(f.x, 1.f + __expf(-zz.x)), __fdividef(f.y, 1.f + __expf(-zz.y)));
  }
  *p = raw;
}

}  // namespace ft

using namespace ft;

extern "C" {

int ft_embed_pair(const int* ids, const int* token_pos, const int* token_seg, const int* seg_slot,
                  const int* seg_q_start, const void* table, const void* pair_table, int* last_token,
                  float* residual, long long slot_stride, long long mul_prev, long long mul_cur, int buckets,
                  int H, int vocab, int copies, float scale, int table_dtype, int T, cudaStream_t stream) {
  if (T <= 0) return FT_OK;
  if (copies < 1 || (pair_table && (buckets < 1 || !last_token))) return FT_ERR_SHAPE;
  EmbedPairArgs a{ids, token_pos, token_seg, seg_slot, seg_q_start, table, pair_table, last_token, residual,
                  slot_stride, mul_prev, mul_cur, buckets, H, vocab, copies, scale};
  FT_DISPATCH(table_dtype, WT, launch_pdl(embed_pair_kernel<WT>, dim3(T), dim3(256), 0, stream, a));
  FT_LAUNCH_CHECK();
  return FT_OK;
}

int ft_embed_norm(const int* ids, const void* table, int table_dtype, const float* weight, float* residual,
                  int T, int H, int vocab, float eps, cudaStream_t stream) {
  if (T <= 0) return FT_OK;
  const bool vec = !(H & 3) && H <= 4 * EMBED_THREADS * EMBED_KEEP && !((uintptr_t)table & 15) &&
                   !((uintptr_t)weight & 15) && !((uintptr_t)residual & 15) &&
                   (table_dtype == FT_DTYPE_F32 || !(H & 7));
  if (vec) {
    FT_DISPATCH(table_dtype, WT,
                (launch_pdl(embed_norm_kernel<WT, true>, dim3(T), dim3(EMBED_THREADS), 0, stream, ids,
                            (const WT*)table, weight, residual, H, vocab, eps)));
  } else {
    FT_DISPATCH(table_dtype, WT,
                (launch_pdl(embed_norm_kernel<WT, false>, dim3(T), dim3(EMBED_THREADS), 0, stream, ids,
                            (const WT*)table, weight, residual, H, vocab, eps)));
  }
  FT_LAUNCH_CHECK();
  return FT_OK;
}

int ft_key_store(const void* src, void* q_out, void* pages, const float* k_weight, const int* token_pos,
                 const int* token_seg, const int* block_table, long long ld, long long page_stride,
                 int q_off, int k_off, int nq, int dq, int nkv, int dk, int P, int table_width, int every,
                 float coef, float eps, int dtype, int T, cudaStream_t stream) {
  if (T <= 0) return FT_OK;
  if (nkv <= 0 || dk <= 0 || P <= 0 || (coef != 0.f && every <= 0)) return FT_ERR_SHAPE;
  KeyStoreArgs a{src, q_out, pages, k_weight, token_pos, token_seg, block_table, ld, page_stride,
                 q_off, k_off, nq, dq, nkv, dk, P, table_width, every, coef, eps};
  // with queries to scale a block takes one token; rows of keys alone are dealt out four tokens a block
  const int per_block = q_out ? 1 : (nkv >= 4 ? 1 : 4 / nkv);
  const dim3 grid((T + per_block - 1) / per_block);
  const bool vec = dtype == FT_DTYPE_BF16 && !(ld & 7) && !(q_off & 7) && !(k_off & 7) && !(dk & 7) &&
                   !((nq * dq) & 7) && !(page_stride & 7) && !((uintptr_t)src & 15) && !((uintptr_t)q_out & 15) &&
                   !((uintptr_t)pages & 15) && !((uintptr_t)k_weight & 15);
  if (vec) {
    launch_pdl(key_store_kernel<__nv_bfloat16, true>, grid, dim3(128), 0, stream, a, T, per_block);
  } else {
    FT_DISPATCH(dtype, AT, (launch_pdl(key_store_kernel<AT, false>, grid, dim3(128), 0, stream, a, T, per_block)));
  }
  FT_LAUNCH_CHECK();
  return FT_OK;
}

int ft_gate_heads(void* o, const void* z, long long ldz, int heads, int d, int dtype, int T, cudaStream_t stream) {
  if (T <= 0) return FT_OK;
  const long long n = (long long)T * heads * d;
  if (dtype == FT_DTYPE_BF16 && d == 1 && !(heads & 7) && !(ldz & 7) && !((uintptr_t)o & 15) && !((uintptr_t)z & 15)) {
    // a gate per value: both rows in 16-byte pieces
    const long long pieces = n >> 3;
    launch_pdl(gate_values_bf16x8_kernel, dim3((unsigned)((pieces + 255) / 256)), dim3(256), 0, stream,
               (__nv_bfloat16*)o, (const __nv_bfloat16*)z, ldz, heads >> 3, pieces);
    FT_LAUNCH_CHECK();
    return FT_OK;
  }
  if (dtype == FT_DTYPE_BF16 && !(d & 7) && !((uintptr_t)o & 15)) {
    const long long pieces = n >> 3;
    launch_pdl(gate_heads_kernel<__nv_bfloat16, 8>, dim3((unsigned)((pieces + 255) / 256)), dim3(256), 0, stream,
               (__nv_bfloat16*)o, (const __nv_bfloat16*)z, ldz, heads, d, pieces);
    FT_LAUNCH_CHECK();
    return FT_OK;
  }
  const unsigned blocks = (unsigned)((n + 255) / 256);
  FT_DISPATCH(dtype, AT,
              (launch_pdl(gate_heads_kernel<AT, 1>, dim3(blocks), dim3(256), 0, stream, (AT*)o, (const AT*)z, ldz,
                          heads, d, n)));
  FT_LAUNCH_CHECK();
  return FT_OK;
}

int ft_activation(void* x, long long n, int kind, int dtype, cudaStream_t stream) {
  if (n <= 0) return FT_OK;
  if (kind < 0 || kind > 2) return FT_ERR_SHAPE;
  if (dtype == FT_DTYPE_BF16 && !(n & 7) && !((uintptr_t)x & 15)) {
    const long long n8 = n >> 3;
    launch_pdl(activation_bf16x8_kernel, dim3((unsigned)((n8 + 255) / 256)), dim3(256), 0, stream, (uint4*)x, n8,
               kind);
    FT_LAUNCH_CHECK();
    return FT_OK;
  }
  FT_DISPATCH(dtype, AT,
              launch_pdl(activation_kernel<AT>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, (AT*)x, n,
                         kind));
  FT_LAUNCH_CHECK();
  return FT_OK;
}

int ft_softcap(float* x, long long n, float cap, cudaStream_t stream) {
  if (n <= 0) return FT_OK;
  if (!(cap > 0.f)) return FT_ERR_SHAPE;
  launch_pdl(softcap_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x, n, cap);
  FT_LAUNCH_CHECK();
  return FT_OK;
}

int ft_norm_add(const void* branch, int k, const float* part_scale, const float* weight, int plus_one, float eps,
                float mult, float* residual, const float* next_weight, int next_plus_one, float next_eps,
                void* next_out, int T, int H, int dtype, cudaStream_t stream) {
  if (T <= 0) return FT_OK;
  if (k <= 0 || H <= 0 || H > 12288) return FT_ERR_SHAPE;
  const bool vec = !(H & 3) && H <= 4 * 256 * NORM_ADD_KEEP && !((uintptr_t)branch & 15) && !((uintptr_t)weight & 15) &&
                   !((uintptr_t)residual & 15) && !((uintptr_t)next_weight & 15) && !((uintptr_t)next_out & 15);
  if (vec) {
    FT_DISPATCH(dtype, AT,
                (launch_pdl(norm_add_kernel<AT, true>, dim3(T), dim3(256), 0, stream, (const AT*)branch, k, part_scale,
                            weight, plus_one, eps, mult, residual, next_weight, next_plus_one, next_eps,
                            (AT*)next_out, H)));
  } else {
    FT_DISPATCH(dtype, AT,
                (launch_pdl(norm_add_kernel<AT, false>, dim3(T), dim3(256), (size_t)H * sizeof(float), stream,
                            (const AT*)branch, k, part_scale, weight, plus_one, eps, mult, residual, next_weight,
                            next_plus_one, next_eps, (AT*)next_out, H)));
  }
  FT_LAUNCH_CHECK();
  return FT_OK;
}

int ft_scaled_sum(const void* parts, const float* scale, void* out, int k, int T, int H, int dtype,
                  cudaStream_t stream) {
  if (T <= 0) return FT_OK;
  const long long n = (long long)T * H;
  FT_DISPATCH(dtype, AT,
              (launch_pdl(scaled_sum_kernel<AT>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream,
                          (const AT*)parts, scale, (AT*)out, k, n, H)));
  FT_LAUNCH_CHECK();
  return FT_OK;
}

int ft_bias_add(void* x, long long ld, const float* bias, int T, int width, int dtype, cudaStream_t stream) {
  if (T <= 0 || width <= 0) return FT_OK;
  const long long n = (long long)T * width;
  FT_DISPATCH(dtype, AT,
              (launch_pdl(bias_add_kernel<AT>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, (AT*)x, ld,
                          bias, n, width)));
  FT_LAUNCH_CHECK();
  return FT_OK;
}

int ft_glu_rows(const void* gu, void* mid, int T, int I, int kind, float alpha, float limit, int dtype,
                cudaStream_t stream) {
  if (T <= 0 || I <= 0) return FT_OK;
  if (kind < 0 || kind > 3) return FT_ERR_SHAPE;
  const long long n = (long long)T * I;
  FT_DISPATCH(dtype, AT,
              (launch_pdl(glu_rows_kernel<AT>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream,
                          (const AT*)gu, (AT*)mid, n, I, kind, alpha, limit)));
  FT_LAUNCH_CHECK();
  return FT_OK;
}

int ft_hyper_norm(float* streams, const void* branch, int k, const float* mix, const float* out_w,
                  const float* read, const float* weight, const float* bias, float eps, int center, void* normed,
                  int T, int S, int H, int dtype, cudaStream_t stream) {
  if (T <= 0) return FT_OK;
  if (S < 1 || S > HYPER_MAX_STREAMS || H <= 0 || H > 10240 || (branch && k <= 0)) return FT_ERR_SHAPE;
  const bool vec = !(H & 3) && H <= 8192 && S <= 4 && !((uintptr_t)streams & 15) && !((uintptr_t)branch & 15) &&
                   !((uintptr_t)weight & 15) && !((uintptr_t)bias & 15) && !((uintptr_t)normed & 15) &&
                   (dtype == FT_DTYPE_F32 || !(H & 7));
  if (vec) {
    cudaError_t e = cudaSuccess;
    FT_DISPATCH(dtype, AT, {
      const AT* b = (const AT*)branch;
      AT* o = (AT*)normed;
      switch (S) {
        case 1: e = launch_hyper_vec<AT, 1>(stream, T, H, streams, b, k, mix, out_w, read, weight, bias, eps, center, o); break;
        case 2: e = launch_hyper_vec<AT, 2>(stream, T, H, streams, b, k, mix, out_w, read, weight, bias, eps, center, o); break;
        case 3: e = launch_hyper_vec<AT, 3>(stream, T, H, streams, b, k, mix, out_w, read, weight, bias, eps, center, o); break;
        default: e = launch_hyper_vec<AT, 4>(stream, T, H, streams, b, k, mix, out_w, read, weight, bias, eps, center, o); break;
      }
    });
    if (e != cudaSuccess) return (int)e;
    FT_LAUNCH_CHECK();
    return FT_OK;
  }
  FT_DISPATCH(dtype, AT,
              (launch_pdl(hyper_norm_kernel<AT>, dim3(T), dim3(256), (size_t)H * sizeof(float), stream, streams,
                          (const AT*)branch, k, mix, out_w, read, weight, bias, eps, center, (AT*)normed, S, H)));
  FT_LAUNCH_CHECK();
  return FT_OK;
}

int ft_rms_rows(const void* x, long long ldx, const float* w, void* out, long long ldo, int T, int n, float eps,
                int dtype, cudaStream_t stream) {
  if (T <= 0) return FT_OK;
  if (n <= 0) return FT_ERR_SHAPE;
  FT_DISPATCH(dtype, AT,
              (launch_pdl(rms_rows_kernel<AT>, dim3(T), dim3(128), 0, stream, (const AT*)x, ldx, w, (AT*)out, ldo, n,
                          eps)));
  FT_LAUNCH_CHECK();
  return FT_OK;
}

int ft_latent_store(const void* down, long long ld_down, const void* q, long long ld_q, void* q_abs, void* pages,
                    long long page_stride, const float* weight, const float* cos_sin, const int* token_pos,
                    const int* token_seg, const int* block_table, int heads, int dq, int rank, int rot, int P,
                    int table_width, int interleaved, float eps, int dtype, int T, cudaStream_t stream) {
  if (T <= 0) return FT_OK;
  if (heads <= 0 || dq < 0 || rank <= 0 || rot < 0 || (rot & 1) || P <= 0) return FT_ERR_SHAPE;
  LatentStoreArgs a{down, q, q_abs, pages, weight, cos_sin, token_pos, token_seg, block_table, ld_down, ld_q,
                    page_stride, heads, dq, rank, rot, P, table_width, interleaved, eps};
  FT_DISPATCH(dtype, AT, (launch_pdl(latent_store_kernel<AT>, dim3(T), dim3(128), 0, stream, a)));
  FT_LAUNCH_CHECK();
  return FT_OK;
}

}  // extern "C"
