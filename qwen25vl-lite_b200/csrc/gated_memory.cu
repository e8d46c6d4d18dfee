// Matrix memories with gates that depend on the token: per head a state S [D, Dv] in float, carried from
// token to token,
//
//     S_t = diag(a_t) S_(t-1) + b_t k_t v_t^T,          o_t = S_t^T q_t.
//
// Two kinds of gate:
//   * per key channel (gated linear attention): a_t [D] comes as a table of decays in (0, 1), b_t = 1;
//   * per head with a running maximum (the matrix memory of xLSTM): from the logarithms i_t, f_t of an input and
//     a forget gate, m_t = max(f_t + m_(t-1), i_t) (m starts at 0), a_t = exp(f_t + m_(t-1) - m_t) for every
//     channel, b_t = exp(i_t - m_t).  The normaliser n_t = a_t n_(t-1) + b_t k_t is one more column of S (its value
//     is 1 for every token), so o_t's last entry is n_t . q_t.  The state keeps m too, as one more row of S.
//
// The walk (memory_scan_kernel): a CTA owns a request's run of tokens, one head and 32 columns of S; a thread
// owns one column's entries in RPT rows, in registers.  The run is taken GM_TOKENS tokens at a time: the tokens' q,
// k, decays and the 32 values are staged in shared memory as floats, every thread walks the tokens without a
// barrier (S never leaves its registers), leaving its part of every o_t in shared memory; then the parts of the row
// slices are added in slice order and o_t goes to memory as floats.  The order of every sum depends on the sizes
// alone, so a token's result does not depend on where its run was cut or on the batch.
//
// Long runs are cut into chunks of tokens that are walked in parallel (the host plans them; `items` then says what
// every CTA row of the grid walks).  Pass 1 walks every chunk from an empty memory (S = 0, m = -inf), without outputs,
// and leaves in scratch the chunk's own sum L, with what the fold needs to carry a state across the chunk: the
// product of the chunk's decays per key channel, or the sum of its log forget gates and its own maximum.
// memory_fold_kernel then goes over a run's chunks in order, an element of S per thread: it leaves every chunk the
// state before it (in place of L) and the request the state after the last one: S <- A S + L per channel, or
// m' = max(F + m, m_L), S <- exp(F + m - m') S + exp(m_L - m') L per head.  Pass 2 walks every chunk again, from the
// state before it, with outputs; runs too short to cut are walked in pass 2 from and to the request's state.  A
// chunk's border moves rounding only: the fold multiplies by the product of the decays where the walk multiplies
// token by token.
//
// The output (memory_output_kernel, a warp per token and head): o_t divided by max(|n_t . q_t|, exp(-m_t)) + 1e-6
// where the memory has a normaliser; divided by its root mean square over the head's Dv channels (eps inside the
// root); times a weight per channel; times silu or sigmoid of the token's gate channel; in T.
//
// Everything here is float but the projections the kernels read (q, k, v, the output gate) and the result.
#include "common.cuh"
#include "row_logits.cuh"

#define GM_TOKENS 16
#define GM_COLS 32
#define GM_FOLD 8           // chunks whose sums a thread of the fold asks for at once

// Four consecutive channels as floats (bf16: 8 bytes, float: 16 bytes at a time).
template <typename T> __device__ __forceinline__ float4 gm_load4(const T* p);
template <> __device__ __forceinline__ float4 gm_load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 gm_load4<bf16>(const bf16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}

__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

// decay[n, c] = sigmoid(z)^(1 / tau), z = bias[c] + sum_r a2t[r, c] * low[n, r]: the low-rank projection's second
// factor (transposed, float), the bias and the map into (0, 1) in one pass; computed as exp(log sigmoid(z) / tau).
// A block takes 8 tokens and as many channels as it has threads, so that a column of a2t read from cache serves
// eight tokens.
template <typename T>
__global__ void gla_decay_kernel(const T* __restrict__ x, int x_stride, int low_off, int rank, const float* __restrict__ a2t,
                                 const float* __restrict__ bias, float inv_tau, float* __restrict__ decay, int n_tokens, int channels) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) float low_s[];     // [8][rank]
  const int n0 = blockIdx.x * 8;
  for (int i = threadIdx.x; i < 8 * rank; i += blockDim.x) {
    const int t = i / rank, r = i % rank;
    low_s[i] = n0 + t < n_tokens ? to_f32(x[(size_t)(n0 + t) * x_stride + low_off + r]) : 0.f;
  }
  __syncthreads();
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
    float z[8];
    const float b = bias ? bias[c] : 0.f;
#pragma unroll
    for (int t = 0; t < 8; ++t) z[t] = b;
    for (int r = 0; r < rank; ++r) {
      const float w = a2t[(size_t)r * channels + c];
#pragma unroll
      for (int t = 0; t < 8; ++t) z[t] = fmaf(w, low_s[t * rank + r], z[t]);
    }
#pragma unroll
    for (int t = 0; t < 8; ++t)
      if (n0 + t < n_tokens) decay[(size_t)(n0 + t) * channels + c] = expf(log_sigmoid(z[t]) * inv_tau);
  }
}

// out[n, j] = bias[j] + w[j, :] . h[n, :] for a few float rows w (gates of a recurrence), float results.
template <typename T, int TOK>
__global__ void __launch_bounds__(256)
row_dots_kernel(const T* __restrict__ h, const float* __restrict__ w, const float* __restrict__ bias, float* __restrict__ out,
                int n_tokens, int hidden, int rows) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) float dots_smem[];
  route_logits<T, TOK>(h, w, nullptr, dots_smem, n_tokens, hidden, rows);
  const float* zs = dots_smem + TOK * ((hidden + 3) & ~3);
  const int n0 = blockIdx.x * TOK;
  for (int i = threadIdx.x; i < TOK * rows; i += 256) {
    const int t = i / rows, j = i % rows;
    if (n0 + t < n_tokens) out[(size_t)(n0 + t) * rows + j] = zs[t * (ROW_LOGITS_MAX + 1) + j] + (bias ? bias[j] : 0.f);
  }
}

struct MemoryArgs {
  const void* x;            // [N, x_stride] in T: q, k, v at their offsets, heads side by side
  int x_stride, q_off, k_off, v_off;
  const float* decay;       // per key channel [N, H * D] (gates per channel), or nullptr
  const float* gates;       // per head [N, 2 * H]: what becomes log i, then what becomes log f (gates per head), or nullptr
  float cap;                // the per-head gates are squashed by cap * tanh(. / cap) first (0: taken as they are)
  float q_scale;
  float* state;             // [slots][H][D + extra][Dv + extra]
  const int* cu_q;
  const int* slot_ids;
  float* o_raw;             // [N, H, Dv + extra]
  float* m_exp;             // [N, H]: exp(-m_t) (gates per head)
  int H, D, Dv, extra;
  // with items: CTA row y walks items[y] = (first token row, end, source, destination, flags) instead of entry y
  const int* items;
  float* scratch;           // [chunks][H][D + extra][Dv + extra]: states between chunks
  float* aux;               // per channel [chunks][H][D]: the product of a chunk's decays; per head [chunks][H][2]: sum of log f, the chunk's own m
};

#define GM_SRC_SCRATCH 1    // the walk starts from scratch[source] (else from the state of entry `source`)
#define GM_DST_NONE 2       // the state after the walk is not kept (else it goes back to where it came from)

// (a, b) stands for x -> max(x + a, b); `first` then `second` is x -> max(x + a1 + a2, max(b1 + a2, b2)).
__device__ __forceinline__ void maxplus_after(float& a, float& b, float a1, float b1) {
  b = fmaxf(b1 + a, b);
  a = a1 + a;
}

// LOCAL: pass 1 of a cut run (from an empty memory, no outputs, the chunk's sum and its carry factors to scratch).
template <typename T, int RPT, bool PER_HEAD, bool LOCAL>
__global__ void memory_scan_kernel(MemoryArgs p) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) float gm_smem[];
  const int DG = blockDim.y, Dp = DG * RPT;
  const int head = blockIdx.x, seq = blockIdx.y;
  const int lane = threadIdx.x, g = threadIdx.y, tid = g * GM_COLS + lane, n_threads = GM_COLS * DG;
  const int cols = p.Dv + p.extra, col0 = blockIdx.z * GM_COLS, col = col0 + lane;
  const bool col_ok = col < cols;
  float* q_s = gm_smem;                                  // [GM_TOKENS][Dp]
  float* k_s = q_s + GM_TOKENS * Dp;
  float* a_s = k_s + GM_TOKENS * Dp;                     // per channel: [GM_TOKENS][Dp]; per head: [GM_TOKENS] a_t, [GM_TOKENS] b_t, m
  float* v_s = a_s + (PER_HEAD ? 2 * GM_TOKENS + 4 : GM_TOKENS * Dp);      // [GM_TOKENS][GM_COLS]
  float* part = v_s + GM_TOKENS * GM_COLS;               // [GM_TOKENS][DG][GM_COLS]
  const size_t st_floats = (size_t)(p.D + p.extra) * cols;
  int begin, end, flags = 0;
  float* st;
  if (p.items) {
    const int* it = p.items + 5 * seq;
    begin = it[0]; end = it[1]; flags = it[4];
    if (LOCAL) st = p.scratch + ((size_t)it[3] * p.H + head) * st_floats;
    else if (flags & GM_SRC_SCRATCH) st = p.scratch + ((size_t)it[2] * p.H + head) * st_floats;
    else st = p.state + ((size_t)p.slot_ids[it[2]] * p.H + head) * st_floats;
  } else {
    begin = p.cu_q[seq]; end = p.cu_q[seq + 1];
    st = p.state + ((size_t)p.slot_ids[seq] * p.H + head) * st_floats;
  }
  const int chunk = p.items ? p.items[5 * seq + 3] : 0;
  // every row of a head is whole and starts where four channels can be read at once
  const bool vec = Dp == p.D && !((p.x_stride | p.q_off | p.k_off | p.D) & 3) && !((uintptr_t)p.x & 15) && !((uintptr_t)p.decay & 15);
  const T* x = (const T*)p.x;

  float S[RPT];
  float P[LOCAL && !PER_HEAD ? RPT : 1];                 // pass 1, decays per channel: their product over the chunk
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int r = g * RPT + i;
    S[i] = (!LOCAL && r < p.D && col_ok) ? st[(size_t)r * cols + col] : 0.f;
    if (LOCAL && !PER_HEAD) P[i] = 1.f;
  }
  // every column keeps a copy of m; the CTA reads its first
  float m_carry = PER_HEAD ? (LOCAL ? -INFINITY : st[(size_t)p.D * cols + col0]) : 0.f;
  float f_sum = 0.f;                                     // pass 1, gates per head: the sum of the chunk's log forget gates

  for (int t0 = begin; t0 < end; t0 += GM_TOKENS) {
    const int nt = min(GM_TOKENS, end - t0);
    __syncthreads();                                     // the chunk before has been read out
    if (vec) {
      // four channels a load
      const int per_row = Dp >> 2;
      for (int i = tid; i < nt * per_row; i += n_threads) {
        const int t = i / per_row, r = (i - t * per_row) << 2;
        const size_t row = (size_t)(t0 + t) * p.x_stride + head * p.D + r;
        if (!LOCAL) {
          float4 q = gm_load4<T>(x + row + p.q_off);
          q.x *= p.q_scale; q.y *= p.q_scale; q.z *= p.q_scale; q.w *= p.q_scale;
          *reinterpret_cast<float4*>(q_s + t * Dp + r) = q;
        }
        *reinterpret_cast<float4*>(k_s + t * Dp + r) = gm_load4<T>(x + row + p.k_off);
        if (!PER_HEAD)
          *reinterpret_cast<float4*>(a_s + t * Dp + r) = *reinterpret_cast<const float4*>(p.decay + ((size_t)(t0 + t) * p.H + head) * p.D + r);
      }
    } else {
      for (int i = tid; i < nt * Dp; i += n_threads) {
        const int t = i / Dp, r = i % Dp;
        const size_t row = (size_t)(t0 + t) * p.x_stride;
        const bool ok = r < p.D;
        if (!LOCAL) q_s[i] = ok ? to_f32(x[row + p.q_off + head * p.D + r]) * p.q_scale : 0.f;
        k_s[i] = ok ? to_f32(x[row + p.k_off + head * p.D + r]) : 0.f;
        if (!PER_HEAD) a_s[i] = ok ? p.decay[((size_t)(t0 + t) * p.H + head) * p.D + r] : 0.f;
      }
    }
    for (int i = tid; i < nt * GM_COLS; i += n_threads) {
      const int t = i / GM_COLS, c = col0 + i % GM_COLS;
      v_s[i] = c < p.Dv ? to_f32(x[(size_t)(t0 + t) * p.x_stride + p.v_off + head * p.Dv + c]) : (c < cols ? 1.f : 0.f);
    }
    if (PER_HEAD && g == 0) {
      // the chunk's gates by the first warp: lane t holds token t's map x -> max(x + f_t, i_t); an inclusive scan composes
      // them, applied to the m that came in it gives every m_t at once
      float li = -INFINITY, lf = 0.f;
      if (lane < nt) {
        const float* gt = p.gates + (size_t)(t0 + lane) * 2 * p.H;
        float zi = gt[head], zf = gt[p.H + head];
        if (p.cap > 0.f) { zi = p.cap * tanhf(zi / p.cap); zf = p.cap * tanhf(zf / p.cap); }
        li = zi;
        lf = log_sigmoid(zf);
      }
      float a = lf, b = li;
#pragma unroll
      for (int o = 1; o < GM_TOKENS; o <<= 1) {
        const float a1 = __shfl_up_sync(0xffffffffu, a, o), b1 = __shfl_up_sync(0xffffffffu, b, o);
        if (lane >= o) maxplus_after(a, b, a1, b1);
      }
      const float m_t = fmaxf(m_carry + a, b);
      float m_prev = __shfl_up_sync(0xffffffffu, m_t, 1);
      if (lane == 0) m_prev = m_carry;
      if (lane < nt) {
        a_s[lane] = expf(lf + m_prev - m_t);
        a_s[GM_TOKENS + lane] = expf(li - m_t);
        if (!LOCAL && blockIdx.z == 0) p.m_exp[(size_t)(t0 + lane) * p.H + head] = expf(-m_t);
      }
      if (lane == nt - 1) { a_s[2 * GM_TOKENS] = m_t; a_s[2 * GM_TOKENS + 1] = a; }       // a: the sum of the batch's log f
    }
    __syncthreads();
    if (PER_HEAD) { m_carry = a_s[2 * GM_TOKENS]; f_sum += a_s[2 * GM_TOKENS + 1]; }
    for (int t = 0; t < nt; ++t) {
      const float4* q4 = reinterpret_cast<const float4*>(q_s + t * Dp + g * RPT);
      const float4* k4 = reinterpret_cast<const float4*>(k_s + t * Dp + g * RPT);
      const float4* a4 = reinterpret_cast<const float4*>(a_s + t * Dp + g * RPT);
      const float v = PER_HEAD ? v_s[t * GM_COLS + lane] * a_s[GM_TOKENS + t] : v_s[t * GM_COLS + lane];
      const float a_head = PER_HEAD ? a_s[t] : 0.f;
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < RPT / 4; ++i) {
        const float4 kk = k4[i];
        float4 qq = make_float4(0.f, 0.f, 0.f, 0.f), aa;
        if (!LOCAL) qq = q4[i];
        if (PER_HEAD) aa = make_float4(a_head, a_head, a_head, a_head);
        else aa = a4[i];
        S[4 * i + 0] = fmaf(aa.x, S[4 * i + 0], kk.x * v);
        S[4 * i + 1] = fmaf(aa.y, S[4 * i + 1], kk.y * v);
        S[4 * i + 2] = fmaf(aa.z, S[4 * i + 2], kk.z * v);
        S[4 * i + 3] = fmaf(aa.w, S[4 * i + 3], kk.w * v);
        if (LOCAL) {
          if (!PER_HEAD) { P[4 * i + 0] *= aa.x; P[4 * i + 1] *= aa.y; P[4 * i + 2] *= aa.z; P[4 * i + 3] *= aa.w; }
        } else {
          acc = fmaf(S[4 * i + 0], qq.x, acc); acc = fmaf(S[4 * i + 1], qq.y, acc);
          acc = fmaf(S[4 * i + 2], qq.z, acc); acc = fmaf(S[4 * i + 3], qq.w, acc);
        }
      }
      if (!LOCAL) part[(t * DG + g) * GM_COLS + lane] = acc;
    }
    __syncthreads();
    if (!LOCAL && col_ok) {
      for (int t = g; t < nt; t += DG) {
        float o = 0.f;
        for (int s = 0; s < DG; ++s) o += part[(t * DG + s) * GM_COLS + lane];
        p.o_raw[((size_t)(t0 + t) * p.H + head) * cols + col] = o;
      }
    }
  }
  if (!LOCAL && (flags & GM_DST_NONE)) return;
  if (col_ok) {
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
      const int r = g * RPT + i;
      if (r < p.D) st[(size_t)r * cols + col] = S[i];
    }
    if (PER_HEAD && g == 0) st[(size_t)p.D * cols + col] = m_carry;
  }
  if (LOCAL && blockIdx.z == 0 && lane == 0) {
    if (PER_HEAD) {
      if (g == 0) { p.aux[((size_t)chunk * p.H + head) * 2] = f_sum; p.aux[((size_t)chunk * p.H + head) * 2 + 1] = m_carry; }
    } else {
#pragma unroll
      for (int i = 0; i < RPT; ++i) {
        const int r = g * RPT + i;
        if (r < p.D) p.aux[((size_t)chunk * p.H + head) * p.D + r] = P[LOCAL && !PER_HEAD ? i : 0];
      }
    }
  }
}

// A run's chunks in order, an element of the state per thread.  runs[y] = (entry, first chunk, chunks).
template <bool PER_HEAD>
__global__ void __launch_bounds__(256) memory_fold_kernel(MemoryArgs p, const int* __restrict__ runs) {
  pdl_trigger();
  pdl_wait();
  const int head = blockIdx.x, cols = p.Dv + p.extra;
  const int* run = runs + 3 * blockIdx.y;
  const int first = run[1], n_chunks = run[2];
  const size_t st_floats = (size_t)(p.D + p.extra) * cols;
  const size_t e = (size_t)blockIdx.z * 256 + threadIdx.x;
  if (e >= st_floats) return;
  const int r = (int)(e / cols);
  float* st = p.state + ((size_t)p.slot_ids[run[0]] * p.H + head) * st_floats;
  float s = st[e];                                        // row D (per head): m, a copy in every column
  float m = PER_HEAD ? st[(size_t)p.D * cols] : 0.f;
  // GM_FOLD chunks at a time: their sums and factors are asked for together, before the first state is written over a
  // sum, so that a thread has that many loads in flight
  for (int c0 = 0; c0 < n_chunks; c0 += GM_FOLD) {
    float local[GM_FOLD], f0[GM_FOLD], f1[GM_FOLD];
#pragma unroll
    for (int i = 0; i < GM_FOLD; ++i) {
      const int c = min(c0 + i, n_chunks - 1);
      local[i] = p.scratch[((size_t)(first + c) * p.H + head) * st_floats + e];
      if (PER_HEAD) {
        const float* ax = p.aux + ((size_t)(first + c) * p.H + head) * 2;
        f0[i] = ax[0]; f1[i] = ax[1];
      } else {
        f0[i] = r < p.D ? p.aux[((size_t)(first + c) * p.H + head) * p.D + r] : 0.f;
        f1[i] = 0.f;
      }
    }
#pragma unroll
    for (int i = 0; i < GM_FOLD; ++i) {
      if (c0 + i < n_chunks) {
        float* sc = p.scratch + ((size_t)(first + c0 + i) * p.H + head) * st_floats;
        if (PER_HEAD) {
          const float f = f0[i], m_local = f1[i];
          const float m_new = fmaxf(f + m, m_local);
          if (r == p.D) {
            sc[e] = m;
            s = m_new;
          } else {
            sc[e] = s;
            s = fmaf(expf(f + m - m_new), s, expf(m_local - m_new) * local[i]);
          }
          m = m_new;
        } else {
          sc[e] = s;
          s = fmaf(f0[i], s, local[i]);
        }
      }
    }
  }
  st[e] = s;
}

// A warp per (token, head).  act: 0 = silu of the gate channel, 1 = sigmoid.
template <typename T>
__global__ void memory_output_kernel(const float* __restrict__ o_raw, const float* __restrict__ m_exp, const T* __restrict__ x,
                                     int x_stride, int g_off, const float* __restrict__ weight, T* __restrict__ out, int n_tokens,
                                     int H, int Dv, int extra, float eps, int act) {
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
  if (item >= (long long)n_tokens * H) return;
  const int n = (int)(item / H), head = (int)(item % H);
  const float* o = o_raw + (size_t)item * (Dv + extra);
  float inv_den = 1.f;
  if (extra) inv_den = 1.0f / (fmaxf(fabsf(o[Dv]), m_exp[item]) + 1e-6f);
  float sq = 0.f;
  for (int c = lane; c < Dv; c += 32) { const float v = o[c] * inv_den; sq = fmaf(v, v, sq); }
  sq = warp_sum(sq);
  const float inv = inv_den / sqrtf(sq / (float)Dv + eps);
  const T* gate = x + (size_t)n * x_stride + g_off + head * Dv;
  T* dst = out + ((size_t)n * H + head) * Dv;
  for (int c = lane; c < Dv; c += 32) {
    const float z = to_f32(gate[c]);
    const float s = 1.0f / (1.0f + expf(-z));
    dst[c] = from_f32<T>(o[c] * inv * weight[head * Dv + c] * (act == 0 ? z * s : s));
  }
}

template <typename T>
static int gla_decay(const void* x, int x_stride, int low_off, int rank, const float* a2t, const float* bias, float tau, float* decay,
                     int n_tokens, int channels, void* stream) {
  if (n_tokens <= 0) return 0;
  if (rank <= 0 || rank > 1024 || !(tau > 0.f)) return (int)cudaErrorInvalidValue;
  const int threads = channels >= 256 ? 256 : 128;
  launch(gla_decay_kernel<T>, dim3((n_tokens + 7) / 8, (channels + threads - 1) / threads), dim3(threads), (size_t)8 * rank * sizeof(float), (cudaStream_t)stream,
         (const T*)x, x_stride, low_off, rank, a2t, bias, 1.0f / tau, decay, n_tokens, channels);
  return launch_status();
}
Q25_EXPORT int q25_memory_gla_decay_f32(const void* x, int xs, int off, int rank, const float* a2t, const float* b, float tau, float* d, int n, int ch, void* s) {
  return gla_decay<float>(x, xs, off, rank, a2t, b, tau, d, n, ch, s);
}
Q25_EXPORT int q25_memory_gla_decay_bf16(const void* x, int xs, int off, int rank, const float* a2t, const float* b, float tau, float* d, int n, int ch, void* s) {
  return gla_decay<bf16>(x, xs, off, rank, a2t, b, tau, d, n, ch, s);
}

template <typename T, int TOK>
static int row_dots_shape(const void* h, const float* w, const float* bias, float* out, int n_tokens, int hidden, int rows, cudaStream_t s) {
  const size_t smem = (size_t)TOK * (((hidden + 3) & ~3) + ROW_LOGITS_MAX + 1) * sizeof(float);
  if (smem > 200 * 1024) return -1;
  if (smem > 48 * 1024) {
    const cudaError_t e = cudaFuncSetAttribute(row_dots_kernel<T, TOK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  launch(row_dots_kernel<T, TOK>, dim3((n_tokens + TOK - 1) / TOK), dim3(256), smem, s, (const T*)h, w, bias, out, n_tokens, hidden, rows);
  return launch_status();
}
template <typename T>
static int row_dots(const void* h, const float* w, const float* bias, float* out, int n_tokens, int hidden, int rows, void* stream) {
  if (n_tokens <= 0) return 0;
  if (rows <= 0 || rows > ROW_LOGITS_MAX) return (int)cudaErrorInvalidValue;
  int rc = -1;
  if (n_tokens >= 512) rc = row_dots_shape<T, 4>(h, w, bias, out, n_tokens, hidden, rows, (cudaStream_t)stream);
  if (rc == -1) rc = row_dots_shape<T, 1>(h, w, bias, out, n_tokens, hidden, rows, (cudaStream_t)stream);
  return rc == -1 ? (int)cudaErrorInvalidValue : rc;
}
Q25_EXPORT int q25_memory_row_dots_f32(const void* h, const float* w, const float* b, float* out, int n, int hidden, int rows, void* s) {
  return row_dots<float>(h, w, b, out, n, hidden, rows, s);
}
Q25_EXPORT int q25_memory_row_dots_bf16(const void* h, const float* w, const float* b, float* out, int n, int hidden, int rows, void* s) {
  return row_dots<bf16>(h, w, b, out, n, hidden, rows, s);
}

template <typename T, int RPT, bool PER_HEAD, bool LOCAL>
static int memory_scan_shape(const MemoryArgs& p, int n_rows, cudaStream_t s) {
  const int DG = (p.D + RPT - 1) / RPT, Dp = DG * RPT;
  const int cols = p.Dv + p.extra;
  const size_t floats = (size_t)2 * GM_TOKENS * Dp + (PER_HEAD ? 2 * GM_TOKENS + 4 : GM_TOKENS * Dp) + GM_TOKENS * GM_COLS +
                        (size_t)GM_TOKENS * DG * GM_COLS;
  const size_t smem = floats * sizeof(float);
  if (smem > 200 * 1024 || DG > 16) return (int)cudaErrorInvalidValue;
  if (smem > 48 * 1024) {
    const cudaError_t e = cudaFuncSetAttribute(memory_scan_kernel<T, RPT, PER_HEAD, LOCAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  launch(memory_scan_kernel<T, RPT, PER_HEAD, LOCAL>, dim3(p.H, n_rows, (cols + GM_COLS - 1) / GM_COLS), dim3(GM_COLS, DG), smem, s, p);
  return launch_status();
}

template <typename T, bool LOCAL>
static int memory_scan_rows(const MemoryArgs& p, int n_rows, cudaStream_t s) {
  if (n_rows <= 0) return 0;
  if (p.extra) {
    if (p.D <= 64) return memory_scan_shape<T, 16, true, LOCAL>(p, n_rows, s);
    if (p.D <= 128) return memory_scan_shape<T, 32, true, LOCAL>(p, n_rows, s);
    return memory_scan_shape<T, 64, true, LOCAL>(p, n_rows, s);
  }
  if (p.D <= 64) return memory_scan_shape<T, 16, false, LOCAL>(p, n_rows, s);
  if (p.D <= 128) return memory_scan_shape<T, 32, false, LOCAL>(p, n_rows, s);
  return memory_scan_shape<T, 64, false, LOCAL>(p, n_rows, s);
}

// per_head 0: decays per key channel from `decay`; 1: gates per head from `gates`, with a normaliser column and m in the state.
template <typename T>
static int memory_scan(const void* x, int x_stride, int q_off, int k_off, int v_off, const float* decay, const float* gates, float cap,
                       float q_scale, float* state, const int* cu_q, const int* slot_ids, float* o_raw, float* m_exp, int n_seqs, int H,
                       int D, int Dv, int per_head, void* stream) {
  if (n_seqs <= 0) return 0;
  if (H <= 0 || D <= 0 || Dv <= 0 || D > 512 || (per_head ? (!gates || !m_exp) : !decay)) return (int)cudaErrorInvalidValue;
  MemoryArgs p;
  p.x = x; p.x_stride = x_stride; p.q_off = q_off; p.k_off = k_off; p.v_off = v_off; p.decay = decay; p.gates = gates; p.cap = cap;
  p.q_scale = q_scale; p.state = state; p.cu_q = cu_q; p.slot_ids = slot_ids; p.o_raw = o_raw; p.m_exp = m_exp;
  p.H = H; p.D = D; p.Dv = Dv; p.extra = per_head ? 1 : 0;
  p.items = nullptr; p.scratch = nullptr; p.aux = nullptr;
  return memory_scan_rows<T, false>(p, n_seqs, (cudaStream_t)stream);
}

// A step with long runs cut into chunks.  first [n_first, 5]: the chunks of pass 1 (token rows, -, chunk, -); runs
// [n_runs, 3]: (entry, first chunk, chunks); second [n_second, 5]: what pass 2 walks, the chunks (from scratch, state not
// kept) and the entries that were not cut (from and to their state).
template <typename T>
static int memory_scan_chunked(const void* x, int x_stride, int q_off, int k_off, int v_off, const float* decay, const float* gates, float cap,
                               float q_scale, float* state, const int* slot_ids, float* o_raw, float* m_exp, const int* first, int n_first,
                               const int* runs, int n_runs, const int* second, int n_second, float* scratch, float* aux, int H, int D, int Dv,
                               int per_head, void* stream) {
  if (H <= 0 || D <= 0 || Dv <= 0 || D > 512 || (per_head ? (!gates || !m_exp) : !decay) || !scratch || !aux) return (int)cudaErrorInvalidValue;
  MemoryArgs p;
  p.x = x; p.x_stride = x_stride; p.q_off = q_off; p.k_off = k_off; p.v_off = v_off; p.decay = decay; p.gates = gates; p.cap = cap;
  p.q_scale = q_scale; p.state = state; p.cu_q = nullptr; p.slot_ids = slot_ids; p.o_raw = o_raw; p.m_exp = m_exp;
  p.H = H; p.D = D; p.Dv = Dv; p.extra = per_head ? 1 : 0; p.scratch = scratch; p.aux = aux;
  cudaStream_t s = (cudaStream_t)stream;
  p.items = first;
  int rc = memory_scan_rows<T, true>(p, n_first, s);
  if (rc) return rc;
  if (n_runs > 0) {
    const size_t st_floats = (size_t)(D + p.extra) * (Dv + p.extra);
    const dim3 grid(H, n_runs, (unsigned)((st_floats + 255) / 256));
    if (per_head) launch(memory_fold_kernel<true>, grid, dim3(256), 0, s, p, runs);
    else launch(memory_fold_kernel<false>, grid, dim3(256), 0, s, p, runs);
    rc = launch_status();
    if (rc) return rc;
  }
  p.items = second;
  return memory_scan_rows<T, false>(p, n_second, s);
}
Q25_EXPORT int q25_memory_scan_chunked_f32(const void* x, int xs, int qo, int ko, int vo, const float* decay, const float* gates, float cap, float qsc,
                                           float* state, const int* slots, float* o_raw, float* m_exp, const int* first, int n_first,
                                           const int* runs, int n_runs, const int* second, int n_second, float* scratch, float* aux, int H, int D,
                                           int Dv, int per_head, void* s) {
  return memory_scan_chunked<float>(x, xs, qo, ko, vo, decay, gates, cap, qsc, state, slots, o_raw, m_exp, first, n_first, runs, n_runs, second,
                                    n_second, scratch, aux, H, D, Dv, per_head, s);
}
Q25_EXPORT int q25_memory_scan_chunked_bf16(const void* x, int xs, int qo, int ko, int vo, const float* decay, const float* gates, float cap, float qsc,
                                            float* state, const int* slots, float* o_raw, float* m_exp, const int* first, int n_first,
                                            const int* runs, int n_runs, const int* second, int n_second, float* scratch, float* aux, int H, int D,
                                            int Dv, int per_head, void* s) {
  return memory_scan_chunked<bf16>(x, xs, qo, ko, vo, decay, gates, cap, qsc, state, slots, o_raw, m_exp, first, n_first, runs, n_runs, second,
                                   n_second, scratch, aux, H, D, Dv, per_head, s);
}
Q25_EXPORT int q25_memory_scan_f32(const void* x, int xs, int qo, int ko, int vo, const float* decay, const float* gates, float cap, float qsc,
                                   float* state, const int* cu, const int* slots, float* o_raw, float* m_exp, int n_seqs, int H, int D, int Dv,
                                   int per_head, void* s) {
  return memory_scan<float>(x, xs, qo, ko, vo, decay, gates, cap, qsc, state, cu, slots, o_raw, m_exp, n_seqs, H, D, Dv, per_head, s);
}
Q25_EXPORT int q25_memory_scan_bf16(const void* x, int xs, int qo, int ko, int vo, const float* decay, const float* gates, float cap, float qsc,
                                    float* state, const int* cu, const int* slots, float* o_raw, float* m_exp, int n_seqs, int H, int D, int Dv,
                                    int per_head, void* s) {
  return memory_scan<bf16>(x, xs, qo, ko, vo, decay, gates, cap, qsc, state, cu, slots, o_raw, m_exp, n_seqs, H, D, Dv, per_head, s);
}

template <typename T>
static int memory_output(const float* o_raw, const float* m_exp, const void* x, int x_stride, int g_off, const float* weight, void* out,
                         int n_tokens, int H, int Dv, int extra, float eps, int act, void* stream) {
  if (n_tokens <= 0) return 0;
  if (extra && !m_exp) return (int)cudaErrorInvalidValue;
  const long long items = (long long)n_tokens * H;
  launch(memory_output_kernel<T>, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, (cudaStream_t)stream, o_raw, m_exp, (const T*)x, x_stride,
         g_off, weight, (T*)out, n_tokens, H, Dv, extra, eps, act);
  return launch_status();
}
Q25_EXPORT int q25_memory_output_f32(const float* o, const float* me, const void* x, int xs, int go, const float* w, void* out, int n, int H, int Dv,
                                     int extra, float eps, int act, void* s) {
  return memory_output<float>(o, me, x, xs, go, w, out, n, H, Dv, extra, eps, act, s);
}
Q25_EXPORT int q25_memory_output_bf16(const float* o, const float* me, const void* x, int xs, int go, const float* w, void* out, int n, int H, int Dv,
                                      int extra, float eps, int act, void* s) {
  return memory_output<bf16>(o, me, x, xs, go, w, out, n, H, Dv, extra, eps, act, s);
}
