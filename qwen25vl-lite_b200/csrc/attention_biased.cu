// Softmax attention over the paged cache with a bias that grows with distance, a sliding window
// beside which the first tokens of the request stay visible, a scale of its own, and values whose
// size may differ from the keys'.  Nothing is rotated here: positions enter through the bias, or the caller
// has turned queries and keys before.
//
//   score(i, j) = (q_i . k_j) * scale - r1[h] * ln(1 + r2[h] * (i - j))        (r1 == nullptr: no bias)
//   query i sees key j when j <= i and (i - j < window or j < keep_first)       (window 0: all j <= i)
//   o_i = softmax_j(score) v_j;  query head h reads kv head h / (nq / nkv)
//   sink[h] (optional): a score without key or value that joins the softmax's denominator
//   dist_bias (optional): a learned table [dist_rows, nq]; score(i, j) += dist_bias[min(i - j, dist_rows - 1), h]
//   gate_off (optional): the token's row holds nq * dv gate channels from that offset on, and
//                        o_i <- o_i * sigmoid(gate_i) channel by channel (an output gate)
//   v_row (optional): values that lie inside the key rows (a latent cache): channels between value rows
//
// and the write of a step's keys and values into their pages, where the values may first be mixed
// with those another layer computed for the same token: v <- (1 - mix) v + mix v_other.
//
// This file holds the general kernels (float or bfloat16, keys of any size, values of up to 512 channels): one warp per
// (token, query head); keys are walked in tiles of 32 aligned to the absolute key index, first the
// kept tokens that the window has left behind, then the window; scores, bias and softmax in float.
// The order of every sum depends on the query's position alone.
#include "common.cuh"
#include "rotary.cuh"

#define BATT_WARPS 4
#define BATT_MAX_D 512

template <typename T>
__global__ void biased_attention_generic_kernel(
    const T* __restrict__ qkv, int qkv_stride, T* __restrict__ out, const T* __restrict__ kpages,
    const T* __restrict__ vpages, const int* __restrict__ block_table, int table_width,
    const int* __restrict__ token_seq, const int* __restrict__ cu_q, const int* __restrict__ q_start_pos,
    int n_tokens, int nq, int nkv, int dk, int dv, int page_size, int window, int keep_first, float scale,
    const float* __restrict__ r1, const float* __restrict__ r2, const float* __restrict__ sink, int v_row, float softcap,
    const float* __restrict__ dist_bias, int dist_rows, int gate_off) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) unsigned char att_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t per_warp = (size_t)(dk + 32) * sizeof(float) + 32 * sizeof(size_t);
  unsigned char* base = att_smem + warp * per_warp;
  size_t* voff = reinterpret_cast<size_t*>(base);
  float* qs = reinterpret_cast<float*>(base + 32 * sizeof(size_t));
  float* ps = qs + dk;

  const long long item = (long long)blockIdx.x * BATT_WARPS + warp;
  if (item >= (long long)n_tokens * nq) return;
  const int token = (int)(item / nq), head = (int)(item % nq);
  const int kvh = head / (nq / nkv);
  const int seq = token_seq[token];
  if (seq < 0) return;
  const int p = q_start_pos[seq] + token - cu_q[seq];
  int lo = window > 0 ? max(0, p - window + 1) : 0;
  if (lo <= keep_first) lo = 0;                       // the kept tokens and the window touch: one range
  const int kept = lo > 0 ? keep_first : 0;           // keys [0, kept) and [lo, p]
  const float b1 = r1 ? r1[head] : 0.f, b2 = r1 ? r2[head] : 0.f;

  const T* q = qkv + (size_t)token * qkv_stride + (size_t)head * dk;
  for (int c = lane; c < dk; c += 32) qs[c] = to_f32(q[c]);
  __syncwarp();

  float m = -INFINITY, l = 0.f;
  float acc[BATT_MAX_D / 32];
#pragma unroll
  for (int i = 0; i < BATT_MAX_D / 32; ++i) acc[i] = 0.f;

  const int* table = block_table + (size_t)seq * table_width;
  for (int range = 0; range < 2; ++range) {
    const int first = range == 0 ? 0 : lo, last = range == 0 ? kept - 1 : p;
    for (int t0 = first & ~31; t0 <= last; t0 += 32) {
      const int key = t0 + lane;
      const bool valid = key >= first && key <= last;
      float s = -INFINITY;
      size_t off = 0;
      if (valid) {
        const int page = table[key / page_size];
        const size_t row = ((size_t)page * nkv + kvh) * page_size + (key % page_size);
        off = row * v_row;
        const T* kr = kpages + row * dk;
        float dot = 0.f;
        for (int c = 0; c < dk; ++c) dot = fmaf(qs[c], to_f32(kr[c]), dot);
        s = dot * scale;
        if (softcap > 0.f) s = softcap * tanhf(s / softcap);      // the scaled score squashed into (-cap, cap)
        if (r1) s -= b1 * log1pf(b2 * (float)(p - key));
        if (dist_bias) s += dist_bias[(size_t)min(p - key, dist_rows - 1) * nq + head];
      }
      const float m_new = fmaxf(m, warp_max(s));  // finite: every tile holds at least one valid key
      const float pexp = valid ? expf(s - m_new) : 0.f;
      const float corr = expf(m - m_new);          // first tile: exp(-inf) = 0
      l = l * corr + warp_sum(pexp);
      m = m_new;
      ps[lane] = pexp;
      voff[lane] = off;
      __syncwarp();
      const int kmax = min(32, last - t0 + 1);
      const int kmin = max(0, first - t0);
#pragma unroll
      for (int i = 0; i < BATT_MAX_D / 32; ++i) {
        const int c = lane + 32 * i;
        if (c < dv) {
          float a = acc[i] * corr;
          for (int kk = kmin; kk < kmax; ++kk) a = fmaf(ps[kk], to_f32(vpages[voff[kk] + c]), a);
          acc[i] = a;
        }
      }
      __syncwarp();
    }
  }
  T* o = out + (size_t)token * nq * dv + (size_t)head * dv;
  if (sink) l += expf(sink[head] - m);                // a score without key or value: it only takes its share of the weight
  const float inv_l = 1.0f / l;
  const T* gate = gate_off >= 0 ? qkv + (size_t)token * qkv_stride + gate_off + (size_t)head * dv : nullptr;
#pragma unroll
  for (int i = 0; i < BATT_MAX_D / 32; ++i) {
    const int c = lane + 32 * i;
    if (c < dv) {
      float v = acc[i] * inv_l;
      if (gate) v *= 1.0f / (1.0f + expf(-to_f32(gate[c])));
      o[c] = from_f32<T>(v);
    }
  }
}

// A step's keys and values into their pages.  qkv rows hold nq*dk query, nkv*dk key and nkv*dv value
// channels.  v_other (row stride ld_other, nkv*dv channels a row; nullptr: none): the values that
// another layer computed for the same tokens, mixed in before the write; the mixed values also
// replace the row's own (the layers that follow may ask for them).
template <typename T>
__global__ void kv_store_mix_kernel(T* __restrict__ qkv, int qkv_stride, const T* __restrict__ v_other, int ld_other, float mix,
                                    T* __restrict__ kpages, T* __restrict__ vpages, const int* __restrict__ kv_slot, int n_tokens,
                                    int nq, int nkv, int dk, int dv, int page_size) {
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x;
  const int slot = kv_slot[n];
  T* row = qkv + (size_t)n * qkv_stride;
  const int k_off = nq * dk, v_off = (nq + nkv) * dk;
  const int page = slot / page_size, in_page = slot % page_size;
  for (int c = threadIdx.x; c < nkv * dk; c += blockDim.x) {
    const int h = c / dk, e = c % dk;
    if (slot >= 0) kpages[(((size_t)page * nkv + h) * page_size + in_page) * dk + e] = row[k_off + c];
  }
  for (int c = threadIdx.x; c < nkv * dv; c += blockDim.x) {
    const int h = c / dv, e = c % dv;
    T v = row[v_off + c];
    if (v_other) {
      v = from_f32<T>(fmaf(mix, to_f32(v_other[(size_t)n * ld_other + c]), (1.0f - mix) * to_f32(v)));
      row[v_off + c] = v;
    }
    if (slot >= 0) vpages[(((size_t)page * nkv + h) * page_size + in_page) * dv + e] = v;
  }
}

template <typename T>
static int biased_attention_generic(const void* qkv, int qkv_stride, void* out, const void* kpages, const void* vpages,
                                    const int* block_table, int table_width, const int* token_seq, const int* cu_q,
                                    const int* q_start_pos, int n_tokens, int nq, int nkv, int dk, int dv, int page_size,
                                    int window, int keep_first, float scale, const float* r1, const float* r2, const float* sink,
                                    int v_row, float softcap, const float* dist_bias, int dist_rows, int gate_off, void* stream) {
  if (n_tokens <= 0) return 0;
  if (v_row <= 0) v_row = dv;
  if (dk <= 0 || dv <= 0 || dv > BATT_MAX_D || dk > 4096 || nkv <= 0 || nq % nkv || window < 0 || keep_first < 0 ||
      (dist_bias && dist_rows < 1))
    return (int)cudaErrorInvalidValue;
  const long long items = (long long)n_tokens * nq;
  const unsigned blocks = (unsigned)((items + BATT_WARPS - 1) / BATT_WARPS);
  const size_t smem = BATT_WARPS * ((size_t)(dk + 32) * sizeof(float) + 32 * sizeof(size_t));
  if (smem > 48 * 1024) {
    const cudaError_t e = cudaFuncSetAttribute(biased_attention_generic_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  launch(biased_attention_generic_kernel<T>, dim3(blocks), dim3(BATT_WARPS * 32), smem, (cudaStream_t)stream, (const T*)qkv,
         qkv_stride, (T*)out, (const T*)kpages, (const T*)vpages, block_table, table_width, token_seq, cu_q, q_start_pos, n_tokens,
         nq, nkv, dk, dv, page_size, window, keep_first, scale, r1, r2, sink, v_row, softcap, dist_bias, dist_rows, gate_off);
  return launch_status();
}

template <typename T>
static int kv_store_mix(void* qkv, int qkv_stride, const void* v_other, int ld_other, float mix, void* kpages, void* vpages,
                        const int* kv_slot, int n_tokens, int nq, int nkv, int dk, int dv, int page_size, void* stream) {
  if (n_tokens <= 0) return 0;
  launch(kv_store_mix_kernel<T>, dim3(n_tokens), dim3(128), 0, (cudaStream_t)stream, (T*)qkv, qkv_stride, (const T*)v_other, ld_other,
         mix, (T*)kpages, (T*)vpages, kv_slot, n_tokens, nq, nkv, dk, dv, page_size);
  return launch_status();
}

Q25_EXPORT int q25_biased_attention_generic_f32(const void* qkv, int qs, void* out, const void* kp, const void* vp, const int* bt,
        int tw, const int* ts, const int* cu, const int* sp, int n, int nq, int nkv, int dk, int dv, int ps, int window, int keep, float scale,
        const float* r1, const float* r2, const float* sink, int v_row, float softcap, const float* db, int db_rows, int gate_off, void* s) {
  return biased_attention_generic<float>(qkv, qs, out, kp, vp, bt, tw, ts, cu, sp, n, nq, nkv, dk, dv, ps, window, keep, scale, r1, r2, sink, v_row, softcap, db, db_rows, gate_off, s);
}
Q25_EXPORT int q25_biased_attention_generic_bf16(const void* qkv, int qs, void* out, const void* kp, const void* vp, const int* bt,
        int tw, const int* ts, const int* cu, const int* sp, int n, int nq, int nkv, int dk, int dv, int ps, int window, int keep, float scale,
        const float* r1, const float* r2, const float* sink, int v_row, float softcap, const float* db, int db_rows, int gate_off, void* s) {
  return biased_attention_generic<bf16>(qkv, qs, out, kp, vp, bt, tw, ts, cu, sp, n, nq, nkv, dk, dv, ps, window, keep, scale, r1, r2, sink, v_row, softcap, db, db_rows, gate_off, s);
}
Q25_EXPORT int q25_kv_store_mix_f32(void* qkv, int qs, const void* vo, int ldo, float mix, void* kp, void* vp, const int* slot, int n,
                                    int nq, int nkv, int dk, int dv, int ps, void* s) {
  return kv_store_mix<float>(qkv, qs, vo, ldo, mix, kp, vp, slot, n, nq, nkv, dk, dv, ps, s);
}
Q25_EXPORT int q25_kv_store_mix_bf16(void* qkv, int qs, const void* vo, int ldo, float mix, void* kp, void* vp, const int* slot, int n,
                                     int nq, int nkv, int dk, int dv, int ps, void* s) {
  return kv_store_mix<bf16>(qkv, qs, vo, ldo, mix, kp, vp, slot, n, nq, nkv, dk, dv, ps, s);
}

// Queries and keys unit-normed per head and turned, keys kept as values: a warp per head, the heads of a token dealt to
// gridDim.y blocks of four warps, so that every head has a warp of its own.
// Row of the token: [nq query heads | nkv key heads] of dk channels each (| nkv value heads of dv channels).  Every
// head is divided by its root mean square (eps inside the root) and multiplied by wq / wk (dk numbers shared by the
// heads); without weights the heads are left as projected, or with unit_norm only divided.  Its first 2 * half
// channels are then turned by the token's angles.  temp_every > 0: the token's queries are multiplied by
// 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1), p its position (a query temperature that grows with the
// context).  Queries are written back in place.  Keys go to their page slot normed and turned; with keys_as_values
// the key as projected (before norm and rotation) is the token's value and goes to the value pages; with dv > 0 the
// row's own values go there.  Statistics, weights, angles and the temperature in float.
template <typename T>
__global__ void qk_norm_store_kernel(T* __restrict__ qk, int qk_stride, const float* __restrict__ wq, const float* __restrict__ wk,
                                     float eps, int unit_norm, const float* __restrict__ angles, int half, int layout,
                                     const int* __restrict__ positions, float temp_coef, int temp_every, T* __restrict__ kpages,
                                     T* __restrict__ vpages, const int* __restrict__ kv_slot, int nq, int nkv, int dk, int dv,
                                     int page_size, int keys_as_values) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) float qkn_smem[];        // a row of dk floats per warp
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
  float* vals = qkn_smem + warp * dk;
  const int n = blockIdx.x;
  const int slot = kv_slot ? kv_slot[n] : -1;
  const int page = slot / page_size, in_page = slot % page_size;
  const float* ang = half > 0 ? angles + (size_t)n * half * 2 : nullptr;
  const float temper = temp_every > 0 ? 1.0f + temp_coef * logf((float)((positions[n] + 1) / temp_every) + 1.0f) : 1.0f;
  for (int head = blockIdx.y * n_warps + warp; head < nq + nkv; head += gridDim.y * n_warps) {
    T* row = qk + (size_t)n * qk_stride + (size_t)head * dk;
    const bool is_key = head >= nq;
    const float* w = is_key ? wk : wq;
    const size_t page_row = is_key ? ((size_t)page * nkv + (head - nq)) * page_size + in_page : 0;
    float sq = 0.f;
    for (int c = lane; c < dk; c += 32) {
      const float v = to_f32(row[c]);
      if (is_key && keys_as_values && slot >= 0) vpages[page_row * dk + c] = row[c];
      sq = fmaf(v, v, sq);
      vals[c] = v;
    }
    sq = warp_sum(sq);
    if (w || unit_norm) {
      const float inv = 1.0f / sqrtf(sq / (float)dk + eps);
      for (int c = lane; c < dk; c += 32) vals[c] = w ? vals[c] * inv * w[c] : vals[c] * inv;
    }
    __syncwarp();
    for (int c = lane; c < dk; c += 32) {
      const float r = rotary_channel<float>(vals, c, half, layout, ang);
      if (is_key) { if (slot >= 0) kpages[page_row * dk + c] = from_f32<T>(r); }
      else row[c] = from_f32<T>(r * temper);
    }
    __syncwarp();
  }
  if (dv > 0 && !keys_as_values && slot >= 0) {
    const T* vrow = qk + (size_t)n * qk_stride + (size_t)(nq + nkv) * dk;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < nkv * dv; c += gridDim.y * blockDim.x)
      vpages[(((size_t)page * nkv + c / dv) * page_size + in_page) * dv + c % dv] = vrow[c];
  }
}

// Four neighbouring channels as they lie in memory, and as floats.
template <typename T> struct Raw4;
template <> struct Raw4<float> { typedef float4 type; };
template <> struct Raw4<bf16> { typedef uint2 type; };
__device__ __forceinline__ float4 raw4_f32(const float4& r) { return r; }
__device__ __forceinline__ float4 raw4_f32(const uint2& r) {
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void f32_raw4(const float4& v, float4& r) { r = v; }
__device__ __forceinline__ void f32_raw4(const float4& v, uint2& r) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  r.x = *reinterpret_cast<const unsigned*>(&a);
  r.y = *reinterpret_cast<const unsigned*>(&b);
}

#define QK_FLAT_CHUNKS 4          // a lane holds up to this many runs of four channels: heads of up to 512 channels

// The same for heads that nothing turns, whose size is a multiple of four (and every row 16 bytes aligned): a warp per
// (token, head), the head's channels in registers, four neighbouring channels a load and a store.  The value heads of a
// row count as heads of their own that are only copied to their page.
template <typename T>
__global__ void qk_norm_store_flat_kernel(T* __restrict__ qk, int qk_stride, const float* __restrict__ wq, const float* __restrict__ wk,
                                          float eps, int unit_norm, const int* __restrict__ positions, float temp_coef, int temp_every,
                                          T* __restrict__ kpages, T* __restrict__ vpages, const int* __restrict__ kv_slot, int n_tokens,
                                          int nq, int nkv, int dk, int dv, int page_size, int keys_as_values) {
  pdl_trigger();
  pdl_wait();
  typedef typename Raw4<T>::type R4;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = nq + nkv + (dv > 0 && !keys_as_values ? nkv : 0);
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
  if (item >= (long long)n_tokens * heads) return;
  const int n = (int)(item / heads), head = (int)(item % heads);
  const int slot = kv_slot ? kv_slot[n] : -1;
  const int page = slot / page_size, in_page = slot % page_size;
  if (head >= nq + nkv) {                                   // a value head: the row's own values to their page
    if (slot < 0) return;
    const int vh = head - nq - nkv;
    const T* src = qk + (size_t)n * qk_stride + (size_t)(nq + nkv) * dk + (size_t)vh * dv;
    T* dst = vpages + (((size_t)page * nkv + vh) * page_size + in_page) * dv;
    if (dv % 4 == 0) {
      for (int c = lane * 4; c < dv; c += 128) *reinterpret_cast<R4*>(dst + c) = *reinterpret_cast<const R4*>(src + c);
    } else {
      for (int c = lane; c < dv; c += 32) dst[c] = src[c];
    }
    return;
  }
  T* row = qk + (size_t)n * qk_stride + (size_t)head * dk;
  const bool is_key = head >= nq;
  const float* w = is_key ? wk : wq;
  const size_t page_row = is_key ? ((size_t)page * nkv + (head - nq)) * page_size + in_page : 0;
  float4 v[QK_FLAT_CHUNKS];
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < QK_FLAT_CHUNKS; ++i) {
    const int c = lane * 4 + 128 * i;
    if (c < dk) {
      const R4 raw = *reinterpret_cast<const R4*>(row + c);
      if (is_key && keys_as_values && slot >= 0) *reinterpret_cast<R4*>(vpages + page_row * dk + c) = raw;
      v[i] = raw4_f32(raw);
      sq = fmaf(v[i].x, v[i].x, sq); sq = fmaf(v[i].y, v[i].y, sq); sq = fmaf(v[i].z, v[i].z, sq); sq = fmaf(v[i].w, v[i].w, sq);
    }
  }
  sq = warp_sum(sq);
  float factor = (w || unit_norm) ? 1.0f / sqrtf(sq / (float)dk + eps) : 1.0f;
  const float temper = !is_key && temp_every > 0 ? 1.0f + temp_coef * logf((float)((positions[n] + 1) / temp_every) + 1.0f) : 1.0f;
  if (is_key && slot < 0) return;
#pragma unroll
  for (int i = 0; i < QK_FLAT_CHUNKS; ++i) {
    const int c = lane * 4 + 128 * i;
    if (c < dk) {
      float4 x = make_float4(v[i].x * factor, v[i].y * factor, v[i].z * factor, v[i].w * factor);
      if (w) { const float4 ww = *reinterpret_cast<const float4*>(w + c); x.x *= ww.x; x.y *= ww.y; x.z *= ww.z; x.w *= ww.w; }
      if (!is_key) { x.x *= temper; x.y *= temper; x.z *= temper; x.w *= temper; }
      R4 raw;
      f32_raw4(x, raw);
      *reinterpret_cast<R4*>(is_key ? kpages + page_row * dk + c : row + c) = raw;
    }
  }
}

template <typename T>
static int qk_norm_store(void* qk, int qk_stride, const float* wq, const float* wk, float eps, int unit_norm, const float* angles, int half,
                         int layout, const int* positions, float temp_coef, int temp_every, void* kpages, void* vpages, const int* kv_slot,
                         int n_tokens, int nq, int nkv, int dk, int dv, int page_size, int keys_as_values, void* stream) {
  if (n_tokens <= 0) return 0;
  if (half < 0 || 2 * half > dk || (layout != ROTARY_INTERLEAVED && layout != ROTARY_HALVES) || (half > 0 && !angles) || dk > 2048 ||
      temp_every < 0 || (temp_every > 0 && !positions) || dv < 0)
    return (int)cudaErrorInvalidValue;
  const int warps = 4;
  const int chunk = 4;                                      // channels of a vector access
  const bool aligned = !(((uintptr_t)qk | (uintptr_t)kpages | (uintptr_t)vpages) & (4 * sizeof(T) - 1)) && !(((uintptr_t)wq | (uintptr_t)wk) & 15);
  if (half == 0 && dk % chunk == 0 && dk <= 128 * QK_FLAT_CHUNKS && qk_stride % chunk == 0 && aligned && (keys_as_values || dv % chunk == 0)) {
    const long long heads = nq + nkv + (dv > 0 && !keys_as_values ? nkv : 0);
    const unsigned blocks = (unsigned)(((long long)n_tokens * heads + 7) / 8);
    launch(qk_norm_store_flat_kernel<T>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, (T*)qk, qk_stride, wq, wk, eps, unit_norm, positions,
           temp_coef, temp_every, (T*)kpages, (T*)vpages, kv_slot, n_tokens, nq, nkv, dk, dv, page_size, keys_as_values);
    return launch_status();
  }
  // as many blocks a token as its heads fill: a warp that walks several heads one after the other waits for each one's loads
  const int per_token = (nq + nkv + warps - 1) / warps;
  launch(qk_norm_store_kernel<T>, dim3(n_tokens, per_token), dim3(warps * 32), (size_t)warps * dk * sizeof(float), (cudaStream_t)stream, (T*)qk,
         qk_stride, wq, wk, eps, unit_norm, angles, half, layout, positions, temp_coef, temp_every, (T*)kpages, (T*)vpages, kv_slot, nq,
         nkv, dk, dv, page_size, keys_as_values);
  return launch_status();
}
Q25_EXPORT int q25_biased_attention_qk_norm_store_f32(void* qk, int qs, const float* wq, const float* wk, float eps, int unit, const float* ang,
        int half, int layout, const int* pos, float tc, int te, void* kp, void* vp, const int* slot, int n, int nq, int nkv, int dk, int dv,
        int ps, int kav, void* s) {
  return qk_norm_store<float>(qk, qs, wq, wk, eps, unit, ang, half, layout, pos, tc, te, kp, vp, slot, n, nq, nkv, dk, dv, ps, kav, s);
}
Q25_EXPORT int q25_biased_attention_qk_norm_store_bf16(void* qk, int qs, const float* wq, const float* wk, float eps, int unit, const float* ang,
        int half, int layout, const int* pos, float tc, int te, void* kp, void* vp, const int* slot, int n, int nq, int nkv, int dk, int dv,
        int ps, int kav, void* s) {
  return qk_norm_store<bf16>(qk, qs, wq, wk, eps, unit, ang, half, layout, pos, tc, te, kp, vp, slot, n, nq, nkv, dk, dv, ps, kav, s);
}

// ================================================================================================
// The bfloat16 tensor-core kernels (mma.sync m16n8k16, float accumulators), FlashAttention-style over
// the pages, for key sizes DK and value sizes DV that are multiples of 16 up to 128.
//
// The keys a piece of work walks are a list of 64-key (runs) or 32-key (single tokens) tiles: first
// the tiles of the kept first tokens that the window has left behind, then the tiles from the
// window's start to the last query; every score is masked by the rule itself (j <= i and (i - j <
// window or j < keep_first)), and a tile of kept tokens counts only keys below keep_first, so no key
// counts twice.  Scores stay in float in the base-2 domain: s = q.k * scale * log2(e) - r1 *
// log2(1 + r2 * (i - j)), one lg2 per score; probabilities are rounded to bfloat16 for P.V only.
//
// Runs: a CTA of 4 warps takes 64 rows of (token, head of the kv group) pairs of one entry and one
// kv head; all warps share the key tiles (two stages of cp.async).  Single tokens: the 4 warps of a
// CTA all hold the token's heads (up to 16) and take the key tiles of their key range in turn, each
// warp with a two-stage pipeline of its own; they merge through shared memory; with more than one
// key range per token (long contexts) the ranges leave (max, sum, unnormalised output) in scratch
// memory and a second kernel adds them up in order.
// ================================================================================================
#include "attention_decode.cuh"

struct BiasedArgs {
  const bf16* qkv;
  int qkv_stride;
  bf16* out;
  const bf16* kpages;
  const bf16* vpages;
  const int* block_table;
  int table_width;
  const int* cu_q;
  const int* q_start_pos;
  const int* items;  // runs: (entry, row tile) pairs; single tokens: entry indices
  int nq, nkv, page_size, window, keep_first;
  float scale_log2;
  float cap_log2, scale_over_cap;   // scores squashed by cap * tanh(q.k * scale / cap): cap * log2(e) and scale / cap (cap_log2 0: not squashed)
  const float* r1;
  const float* r2;
  const float* sink;   // per query head, a score without key or value that joins the denominator (nullptr: none)
  int v_row;           // channels between two value rows of a page (DV, or the key row's when values lie inside the keys)
  const float* dist_bias;  // [dist_rows, nq] added to the score by distance, the last row for every distance beyond (nullptr: none)
  int dist_rows;
  int gate_off;        // where a token's row holds its nq * DV output-gate channels (-1: no gate)
  int n_splits;
  float* part_o;   // [items, nq, splits, DV]
  float* part_ml;  // [items, nq, splits, 2]
};

// sigmoid of two neighbouring gate channels (an even channel offset: one 32-bit load).
__device__ __forceinline__ float2 gate_pair(const bf16* g) {
  const float2 z = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(g));
  return make_float2(1.0f / (1.0f + __expf(-z.x)), 1.0f / (1.0f + __expf(-z.y)));
}
__device__ __forceinline__ float gate_one(const bf16* g) { return 1.0f / (1.0f + __expf(-__bfloat162float(*g))); }

// The tiles of keys that queries at positions p_first .. p_last walk.
struct KeyWalk {
  int kept, lo, hi, sink_tiles, win_key0, n_tiles;
  __device__ __forceinline__ void set(int p_first, int p_last, int window, int keep_first, int bn) {
    lo = window > 0 ? max(0, p_first - window + 1) : 0;
    if (lo <= keep_first) lo = 0;
    kept = lo > 0 ? keep_first : 0;
    hi = p_last;
    sink_tiles = (kept + bn - 1) / bn;
    win_key0 = lo / bn * bn;
    n_tiles = sink_tiles + (hi - win_key0) / bn + 1;
  }
  // first key of tile i, and the range of keys [rl, rh] that count in it
  __device__ __forceinline__ void tile(int i, int bn, int& key0, int& rl, int& rh) const {
    if (i < sink_tiles) { key0 = i * bn; rl = 0; rh = kept - 1; }
    else { key0 = win_key0 + (i - sink_tiles) * bn; rl = lo; rh = hi; }
  }
};

// Copies keys [key0, key0 + BN) of one kv head into K and V tiles (zeros past `last`), by NT threads:
// NT / BN threads share a key, so a thread looks one page up and takes that row's 16-byte chunks
// (of the key and of the value) in turn.
template <int DK, int DV, int BN, int NT>
__device__ __forceinline__ void biased_load_tile(unsigned char* ks, unsigned char* vs, const BiasedArgs& a, const int* table, int kvh,
                                                 int key0, int last, int tid) {
  constexpr int CK = DK / 8, CV = DV / 8, TPK = NT / BN;
  static_assert(NT % BN == 0 && CK % TPK == 0 && CV % TPK == 0, "the chunks of a row divide among its threads");
  const int key = tid / TPK, part = tid % TPK;
  const int kidx = key0 + key;
  const bool valid = kidx <= last;
  const int kc = valid ? kidx : last;                       // a readable address also for the zero-filled rows
  const int page = table[kc / a.page_size];
  const size_t row = ((size_t)page * a.nkv + kvh) * a.page_size + kc % a.page_size;
  const bf16* kr = a.kpages + row * DK;
  const bf16* vr = a.vpages + row * a.v_row;
#pragma unroll
  for (int i = 0; i < CK / TPK; ++i) {
    const int ch = part + i * TPK;
    cp_async16(ks + key * Tile<DK>::PITCH + ch * 16, kr + ch * 8, valid);
  }
#pragma unroll
  for (int i = 0; i < CV / TPK; ++i) {
    const int ch = part + i * TPK;
    cp_async16(vs + key * Tile<DV>::PITCH + ch * 16, vr + ch * 8, valid);
  }
}

// One tile of keys for the warp's 16 rows.  p0/p1: positions of rows g and g+8 (-1: no such row);
// b1x/b2x: the bias numbers of the rows' heads; [rl, rh]: the keys of the tile that count.  FULL: the
// caller has seen that every key of the tile counts for every row of the warp, so nothing is masked.
// TABLE: the rows' heads add tab0 / tab1 [min(distance, dist_rows - 1) * nq] to their scores (a build of
// its own, so that the kernels without a table carry none of it).
template <int DK, int DV, int BN, bool FULL, bool TABLE>
__device__ __forceinline__ void biased_tile(const unsigned (&qf)[DK / 16][4], const unsigned char* ks, const unsigned char* vs,
                                            int key0, int rl, int rh, int p0, int p1, int window, int keep_first, float scale_log2,
                                            float cap_log2, float scale_over_cap, float b10, float b20, float b11, float b21,
                                            const float* __restrict__ tab0, const float* __restrict__ tab1, int dist_rows, int nq,
                                            float (&m)[2], float (&l)[2], float (&o)[DV / 8][4]) {
  constexpr int PK = Tile<DK>::PITCH, PV = Tile<DV>::PITCH;
  const int lane = threadIdx.x & 31, t = lane & 3;
  float s[BN / 8][4];
#pragma unroll
  for (int j = 0; j < BN / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
  for (int kk = 0; kk < DK / 16; ++kk) {
    unsigned b[BN / 8][2];
#pragma unroll
    for (int j = 0; j < BN / 8; ++j) ldmatrix_x2(b[j], ks + (j * 8 + (lane & 7)) * PK + (kk * 16 + 8 * ((lane >> 3) & 1)) * 2);
#pragma unroll
    for (int j = 0; j < BN / 8; ++j) mma_bf16(s[j], qf[kk], b[j][0], b[j][1]);
  }
  // distance of the row's query to the thread's first key of the tile, as a float; the other keys
  // of the thread lie constants further on
  const float d0 = (float)(p0 - key0 - 2 * t), d1 = (float)(p1 - key0 - 2 * t);
  // the distance table: a row whose nearest key of the tile lies at the table's last row or beyond adds one number
  // to all its scores; the table's entries are natural-log scores, the kernel's live in the base-2 domain
  constexpr float LOG2E = 1.4426950408889634f;
  const int last_row = dist_rows - 1;
  const bool far0 = TABLE && p0 - (key0 + BN - 1) >= last_row, far1 = TABLE && p1 - (key0 + BN - 1) >= last_row;
  const float fb0 = far0 ? tab0[(size_t)last_row * nq] * LOG2E : 0.f, fb1 = far1 ? tab1[(size_t)last_row * nq] * LOG2E : 0.f;
  float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
  for (int j = 0; j < BN / 8; ++j) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float fd = (e < 2 ? d0 : d1) - (float)(j * 8 + (e & 1));
      const float b1 = e < 2 ? b10 : b11, b2 = e < 2 ? b20 : b21;
      float v = cap_log2 > 0.f ? cap_log2 * tanhf(s[j][e] * scale_over_cap) - b1 * __log2f(fmaf(b2, fd, 1.0f))
                               : fmaf(s[j][e], scale_log2, -b1 * __log2f(fmaf(b2, fd, 1.0f)));
      if (TABLE) {
        if (e < 2 ? far0 : far1) {
          v += e < 2 ? fb0 : fb1;
        } else {
          const int dist = (e < 2 ? p0 : p1) - (key0 + j * 8 + 2 * t + (e & 1));
          v = fmaf((e < 2 ? tab0 : tab1)[(size_t)min(max(dist, 0), last_row) * nq], LOG2E, v);
        }
      }
      if (!FULL) {
        const int kidx = key0 + j * 8 + 2 * t + (e & 1);
        const int dist = (e < 2 ? p0 : p1) - kidx;
        const bool ok = kidx >= rl && kidx <= rh && dist >= 0 && (window <= 0 || dist < window || kidx < keep_first);
        v = ok ? v : -INFINITY;
      }
      s[j][e] = v;
    }
    mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
    mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
  }
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
  const float mn0 = fmaxf(m[0], mx0), mn1 = fmaxf(m[1], mx1);
  const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;  // nothing seen yet
  const float c0 = exp2f(m[0] - ms0), c1 = exp2f(m[1] - ms1);
  m[0] = mn0;
  m[1] = mn1;
  float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
  for (int j = 0; j < BN / 8; ++j) {
    s[j][0] = exp2f(s[j][0] - ms0);
    s[j][1] = exp2f(s[j][1] - ms0);
    s[j][2] = exp2f(s[j][2] - ms1);
    s[j][3] = exp2f(s[j][3] - ms1);
    sum0 += s[j][0] + s[j][1];
    sum1 += s[j][2] + s[j][3];
  }
  l[0] = l[0] * c0 + sum0;  // per-thread partial sums; the quad is reduced once at the end
  l[1] = l[1] * c1 + sum1;
#pragma unroll
  for (int nb = 0; nb < DV / 8; ++nb) {
    o[nb][0] *= c0;
    o[nb][1] *= c0;
    o[nb][2] *= c1;
    o[nb][3] *= c1;
  }
#pragma unroll
  for (int kk = 0; kk < BN / 16; ++kk) {
    unsigned pa[4];
    pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
    pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
    pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
    const unsigned char* vrow = vs + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * PV;
#pragma unroll
    for (int np = 0; np < DV / 16; ++np) {
      unsigned b[4];
      ldmatrix_x4_trans(b, vrow + (np * 16 + 8 * (lane >> 4)) * 2);
      mma_bf16(o[2 * np], pa, b[0], b[1]);
      mma_bf16(o[2 * np + 1], pa, b[2], b[3]);
    }
  }
}

// Whether every key of the tile [key0, key0 + bn) counts for every query of positions p_min .. p_max.
__device__ __forceinline__ bool tile_is_full(int key0, int bn, int rl, int rh, int p_min, int p_max, int window, int keep_first) {
  const int last = key0 + bn - 1;
  return p_min >= 0 && last <= p_min && key0 >= rl && last <= rh && (window <= 0 || p_max - key0 < window || last < keep_first);
}

// EXTRA: what a build carries beyond scores, masks and sinks: 0 nothing, 1 the output gate, 2 the gate and the distance
// table (kernels of models that have neither are built without a trace of them).
template <int DK, int DV, int EXTRA>
__global__ void __launch_bounds__(128) biased_prefill_kernel(BiasedArgs a) {
  constexpr bool TABLE = EXTRA == 2, GATE = EXTRA >= 1;
  pdl_trigger();
  pdl_wait();
  constexpr int BN = 64, KT = BN * Tile<DK>::PITCH, VT = BN * Tile<DV>::PITCH;
  extern __shared__ __align__(16) unsigned char smem[];     // two stages of (K tile, V tile)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int entry = a.items[2 * blockIdx.x], row_tile = a.items[2 * blockIdx.x + 1];
  const int kvh = blockIdx.y;
  const int group = a.nq / a.nkv;
  const int first = a.cu_q[entry], n = a.cu_q[entry + 1] - first, start = a.q_start_pos[entry];
  const int rows = n * group;
  const int tile_row0 = row_tile * 64;
  const int t_first = tile_row0 / group, t_last = min(tile_row0 + 63, rows - 1) / group;
  KeyWalk walk;
  walk.set(start + t_first, start + t_last, a.window, a.keep_first, BN);
  const int* table = a.block_table + (size_t)entry * a.table_width;
  // this thread's two rows
  const int r0 = tile_row0 + warp * 16 + g, r1 = r0 + 8;
  const int tok0 = r0 < rows ? r0 / group : -1, tok1 = r1 < rows ? r1 / group : -1;
  const int h0 = kvh * group + (r0 < rows ? r0 % group : 0), h1 = kvh * group + (r1 < rows ? r1 % group : 0);
  const int p0 = tok0 < 0 ? -1 : start + tok0, p1 = tok1 < 0 ? -1 : start + tok1;
  const float b10 = a.r1 ? a.r1[h0] : 0.f, b20 = a.r1 ? a.r2[h0] : 0.f, b11 = a.r1 ? a.r1[h1] : 0.f, b21 = a.r1 ? a.r2[h1] : 0.f;
  const float* tab0 = TABLE ? a.dist_bias + h0 : nullptr;
  const float* tab1 = TABLE ? a.dist_bias + h1 : nullptr;
  unsigned qf[DK / 16][4];
  load_q<DK>(qf, [&](int r) -> const bf16* {
    const int rr = tile_row0 + warp * 16 + r;
    return rr < rows ? a.qkv + (size_t)(first + rr / group) * a.qkv_stride + (size_t)(kvh * group + rr % group) * DK : nullptr;
  });
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[DV / 8][4];
#pragma unroll
  for (int i = 0; i < DV / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  // the positions of the warp's 16 rows: the first and the last one (-1 when the warp has rows past the end)
  const int w_row0 = tile_row0 + warp * 16;
  const int wp_min = w_row0 + 15 < rows ? start + w_row0 / group : -1, wp_max = start + min(w_row0 + 15, rows - 1) / group;

  int key0, rl, rh;
  walk.tile(0, BN, key0, rl, rh);
  biased_load_tile<DK, DV, BN, 128>(smem, smem + KT, a, table, kvh, key0, walk.hi, threadIdx.x);
  cp_async_commit();
  for (int i = 0; i < walk.n_tiles; ++i) {
    unsigned char* cur = smem + (i & 1) * (KT + VT);
    if (i + 1 < walk.n_tiles) {
      int nk0, nrl, nrh;
      walk.tile(i + 1, BN, nk0, nrl, nrh);
      unsigned char* nxt = smem + ((i + 1) & 1) * (KT + VT);
      biased_load_tile<DK, DV, BN, 128>(nxt, nxt + KT, a, table, kvh, nk0, walk.hi, threadIdx.x);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    walk.tile(i, BN, key0, rl, rh);
    if (tile_is_full(key0, BN, rl, rh, wp_min, wp_max, a.window, a.keep_first))
      biased_tile<DK, DV, BN, true, TABLE>(qf, cur, cur + KT, key0, rl, rh, p0, p1, a.window, a.keep_first, a.scale_log2, a.cap_log2, a.scale_over_cap, b10, b20, b11, b21, tab0, tab1, a.dist_rows, a.nq, m, l, o);
    else
      biased_tile<DK, DV, BN, false, TABLE>(qf, cur, cur + KT, key0, rl, rh, p0, p1, a.window, a.keep_first, a.scale_log2, a.cap_log2, a.scale_over_cap, b10, b20, b11, b21, tab0, tab1, a.dist_rows, a.nq, m, l, o);
    __syncthreads();
  }
  float l0 = quad_sum(l[0]), l1 = quad_sum(l[1]);
  if (a.sink) {                                              // scores live in the base-2 domain
    if (tok0 >= 0) l0 += exp2f(a.sink[h0] * 1.4426950408889634f - m[0]);
    if (tok1 >= 0) l1 += exp2f(a.sink[h1] * 1.4426950408889634f - m[1]);
  }
  const float i0 = l0 > 0.f ? 1.0f / l0 : 0.f, i1 = l1 > 0.f ? 1.0f / l1 : 0.f;
  const bf16* g0 = GATE && a.gate_off >= 0 && tok0 >= 0 ? a.qkv + (size_t)(first + tok0) * a.qkv_stride + a.gate_off + (size_t)h0 * DV : nullptr;
  const bf16* g1 = GATE && a.gate_off >= 0 && tok1 >= 0 ? a.qkv + (size_t)(first + tok1) * a.qkv_stride + a.gate_off + (size_t)h1 * DV : nullptr;
#pragma unroll
  for (int nb = 0; nb < DV / 8; ++nb) {
    const int c = nb * 8 + 2 * t;
    float y0 = o[nb][0] * i0, y1 = o[nb][1] * i0, y2 = o[nb][2] * i1, y3 = o[nb][3] * i1;
    if (GATE) {
      if (g0) { const float2 z = gate_pair(g0 + c); y0 *= z.x; y1 *= z.y; }
      if (g1) { const float2 z = gate_pair(g1 + c); y2 *= z.x; y3 *= z.y; }
    }
    if (tok0 >= 0) *reinterpret_cast<unsigned*>(a.out + (size_t)(first + tok0) * a.nq * DV + (size_t)h0 * DV + c) = pack_bf16(y0, y1);
    if (tok1 >= 0) *reinterpret_cast<unsigned*>(a.out + (size_t)(first + tok1) * a.nq * DV + (size_t)h1 * DV + c) = pack_bf16(y2, y3);
  }
}

// Single tokens: blockIdx.x = item, blockIdx.y = kv head, blockIdx.z = key range.
template <int DK, int DV, int EXTRA>
__global__ void __launch_bounds__(128) biased_decode_kernel(BiasedArgs a) {
  constexpr bool TABLE = EXTRA == 2, GATE = EXTRA >= 1;
  pdl_trigger();
  pdl_wait();
  constexpr int BN = 32, KT = BN * Tile<DK>::PITCH, VT = BN * Tile<DV>::PITCH, WARP_BYTES = 2 * (KT + VT);
  constexpr int SLAB = DV + 4;                               // floats per merged row
  extern __shared__ __align__(16) unsigned char smem[];     // per warp two stages of (K, V); reused for the merge
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int item = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int entry = a.items[item];
  const int group = a.nq / a.nkv;
  const int token = a.cu_q[entry], p = a.q_start_pos[entry];
  KeyWalk walk;
  walk.set(p, p, a.window, a.keep_first, BN);
  const int per = (walk.n_tiles + a.n_splits - 1) / a.n_splits;
  const int t_begin = split * per, t_end = min(walk.n_tiles, t_begin + per);
  const int* table = a.block_table + (size_t)entry * a.table_width;
  const int h0 = kvh * group + (g < group ? g : 0), h1 = kvh * group + (g + 8 < group ? g + 8 : 0);
  const int p0 = g < group ? p : -1, p1 = g + 8 < group ? p : -1;
  const float b10 = a.r1 ? a.r1[h0] : 0.f, b20 = a.r1 ? a.r2[h0] : 0.f, b11 = a.r1 ? a.r1[h1] : 0.f, b21 = a.r1 ? a.r2[h1] : 0.f;
  const float* tab0 = TABLE ? a.dist_bias + h0 : nullptr;
  const float* tab1 = TABLE ? a.dist_bias + h1 : nullptr;
  unsigned qf[DK / 16][4];
  load_q<DK>(qf, [&](int r) -> const bf16* {
    return r < group ? a.qkv + (size_t)token * a.qkv_stride + (size_t)(kvh * group + r) * DK : nullptr;
  });
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[DV / 8][4];
#pragma unroll
  for (int i = 0; i < DV / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  unsigned char* mine = smem + warp * WARP_BYTES;
  int key0, rl, rh;
  int i = t_begin + warp;
  if (i < t_end) {
    walk.tile(i, BN, key0, rl, rh);
    biased_load_tile<DK, DV, BN, 32>(mine, mine + KT, a, table, kvh, key0, walk.hi, lane);
  }
  cp_async_commit();
  for (int stage = 0; i < t_end; i += 4, stage ^= 1) {
    unsigned char* cur = mine + stage * (KT + VT);
    if (i + 4 < t_end) {
      int nk0, nrl, nrh;
      walk.tile(i + 4, BN, nk0, nrl, nrh);
      unsigned char* nxt = mine + (stage ^ 1) * (KT + VT);
      biased_load_tile<DK, DV, BN, 32>(nxt, nxt + KT, a, table, kvh, nk0, walk.hi, lane);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncwarp();
    walk.tile(i, BN, key0, rl, rh);
    biased_tile<DK, DV, BN, false, TABLE>(qf, cur, cur + KT, key0, rl, rh, p0, p1, a.window, a.keep_first, a.scale_log2, a.cap_log2, a.scale_over_cap, b10, b20, b11, b21, tab0, tab1, a.dist_rows, a.nq, m, l, o);
    __syncwarp();
  }
  cp_async_wait<0>();
  __syncthreads();                                           // every warp is done with its tiles
  // the warps' (max, sum, output) side by side, then each thread merges some (row, column) pairs
  float* ml = reinterpret_cast<float*>(smem);                // [4 warps][16 rows][2]
  float* slab = ml + 4 * 16 * 2;                             // [4 warps][16 rows][SLAB]
  const float l0 = quad_sum(l[0]), l1 = quad_sum(l[1]);
  if (t == 0) {
    ml[(warp * 16 + g) * 2] = m[0]; ml[(warp * 16 + g) * 2 + 1] = l0;
    ml[(warp * 16 + g + 8) * 2] = m[1]; ml[(warp * 16 + g + 8) * 2 + 1] = l1;
  }
#pragma unroll
  for (int nb = 0; nb < DV / 8; ++nb) {
    const int c = nb * 8 + 2 * t;
    slab[(warp * 16 + g) * SLAB + c] = o[nb][0];
    slab[(warp * 16 + g) * SLAB + c + 1] = o[nb][1];
    slab[(warp * 16 + g + 8) * SLAB + c] = o[nb][2];
    slab[(warp * 16 + g + 8) * SLAB + c + 1] = o[nb][3];
  }
  __syncthreads();
  for (int x = threadIdx.x; x < group * DV; x += 128) {
    const int r = x / DV, c = x % DV;
    float mm = -INFINITY;
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, ml[(w * 16 + r) * 2]);
    float sum = 0.f, acc = 0.f;
    for (int w = 0; w < 4; ++w) {
      const float mw = ml[(w * 16 + r) * 2];
      const float f = mw == -INFINITY ? 0.f : exp2f(mw - mm);
      sum = fmaf(ml[(w * 16 + r) * 2 + 1], f, sum);
      acc = fmaf(slab[(w * 16 + r) * SLAB + c], f, acc);
    }
    const int head = kvh * group + r;
    if (a.n_splits == 1) {
      if (a.sink && mm != -INFINITY) sum += exp2f(a.sink[head] * 1.4426950408889634f - mm);
      float y = sum > 0.f ? acc / sum : 0.f;
      if (GATE && a.gate_off >= 0) y *= gate_one(a.qkv + (size_t)token * a.qkv_stride + a.gate_off + (size_t)head * DV + c);
      a.out[(size_t)token * a.nq * DV + (size_t)head * DV + c] = __float2bfloat16_rn(y);
    } else {
      const size_t at = ((size_t)item * a.nq + head) * a.n_splits + split;
      a.part_o[at * DV + c] = acc;
      if (c == 0) { a.part_ml[at * 2] = mm; a.part_ml[at * 2 + 1] = sum; }
    }
  }
}

// Adds the key ranges of a token's head up, in order.  One block per (item, head), DV threads.
template <int DV>
__global__ void biased_combine_kernel(BiasedArgs a) {
  pdl_trigger();
  pdl_wait();
  const int item = blockIdx.x, head = blockIdx.y, c = threadIdx.x;
  const int token = a.cu_q[a.items[item]];
  const size_t base = ((size_t)item * a.nq + head) * a.n_splits;
  float mm = -INFINITY;
  for (int s = 0; s < a.n_splits; ++s) mm = fmaxf(mm, a.part_ml[(base + s) * 2]);
  float sum = 0.f, acc = 0.f;
  for (int s = 0; s < a.n_splits; ++s) {
    const float ms = a.part_ml[(base + s) * 2];
    const float f = ms == -INFINITY ? 0.f : exp2f(ms - mm);
    sum = fmaf(a.part_ml[(base + s) * 2 + 1], f, sum);
    acc = fmaf(a.part_o[(base + s) * DV + c], f, acc);
  }
  if (a.sink && mm != -INFINITY) sum += exp2f(a.sink[head] * 1.4426950408889634f - mm);
  float y = sum > 0.f ? acc / sum : 0.f;
  if (a.gate_off >= 0) y *= gate_one(a.qkv + (size_t)token * a.qkv_stride + a.gate_off + (size_t)head * DV + c);
  a.out[(size_t)token * a.nq * DV + (size_t)head * DV + c] = __float2bfloat16_rn(y);
}

template <int DK, int DV, int EXTRA>
static int biased_mma_launch(const BiasedArgs& a, int n_tiles, int n_items, const int* tiles, const int* items, cudaStream_t s) {
  if (n_tiles > 0) {
    constexpr int SMEM = 2 * 64 * (Tile<DK>::PITCH + Tile<DV>::PITCH);
    if (SMEM > 48 * 1024) {
      const cudaError_t e = cudaFuncSetAttribute(biased_prefill_kernel<DK, DV, EXTRA>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
      if (e != cudaSuccess) return (int)e;
    }
    BiasedArgs b = a;
    b.items = tiles;
    launch(biased_prefill_kernel<DK, DV, EXTRA>, dim3(n_tiles, a.nkv), dim3(128), SMEM, s, b);
  }
  if (n_items > 0) {
    constexpr int TILES = 4 * 2 * 32 * (Tile<DK>::PITCH + Tile<DV>::PITCH), MERGE = (4 * 16 * 2 + 4 * 16 * (DV + 4)) * 4;
    constexpr int SMEM = TILES > MERGE ? TILES : MERGE;
    if (SMEM > 48 * 1024) {
      const cudaError_t e = cudaFuncSetAttribute(biased_decode_kernel<DK, DV, EXTRA>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
      if (e != cudaSuccess) return (int)e;
    }
    BiasedArgs b = a;
    b.items = items;
    launch(biased_decode_kernel<DK, DV, EXTRA>, dim3(n_items, a.nkv, a.n_splits), dim3(128), SMEM, s, b);
    if (a.n_splits > 1) launch(biased_combine_kernel<DV>, dim3(n_items, a.nq), dim3(DV), 0, s, b);
  }
  return launch_status();
}

// Sizes the tensor-core kernels are built for: keys and values of 32, 64 or 128 channels in any pairing, and
// the rows of a latent cache (keys of a rank plus rotated channels over values of the rank alone):
// 48 / 32, 80 / 64, 96 / 64, 160 / 128, 192 / 128.
#define BIASED_SIZES(X) \
  X(32, 32) X(32, 64) X(32, 128) X(64, 32) X(64, 64) X(64, 128) X(128, 32) X(128, 64) X(128, 128) \
  X(48, 32) X(80, 64) X(96, 64) X(160, 128) X(192, 128)
Q25_EXPORT int q25_biased_attention_mma_supports(int dk, int dv) {
#define BIASED_CASE(K, V) if (dk == K && dv == V) return 1;
  BIASED_SIZES(BIASED_CASE)
#undef BIASED_CASE
  return 0;
}

// tiles: (entry, row tile of 64 rows) pairs of the runs; items: the entries of one token (groups of
// up to 16 query heads).  n_splits key ranges per single token; scratch as biased_decode_kernel says.
Q25_EXPORT int q25_biased_attention_mma_bf16(const void* qkv, int qkv_stride, void* out, const void* kp, const void* vp, const int* bt,
                                             int tw, const int* cu, const int* sp, const int* tiles, int n_tiles, const int* items,
                                             int n_items, int nq, int nkv, int dk, int dv, int ps, int window, int keep, float scale,
                                             const float* r1, const float* r2, const float* sink, int v_row, int n_splits, float* part_o,
                                             float* part_ml, float softcap, const float* dist_bias, int dist_rows, int gate_off,
                                             void* stream) {
  if (n_tiles <= 0 && n_items <= 0) return 0;
  if (nkv <= 0 || nq % nkv || ps <= 0 || n_splits < 1 || (n_items > 0 && nq / nkv > 16) || v_row % 8 || (dist_bias && dist_rows < 1) ||
      (gate_off >= 0 && gate_off % 2))
    return (int)cudaErrorInvalidValue;
  BiasedArgs a;
  a.qkv = (const bf16*)qkv; a.qkv_stride = qkv_stride; a.out = (bf16*)out; a.kpages = (const bf16*)kp; a.vpages = (const bf16*)vp;
  a.block_table = bt; a.table_width = tw; a.cu_q = cu; a.q_start_pos = sp; a.items = nullptr;
  a.nq = nq; a.nkv = nkv; a.page_size = ps; a.window = window; a.keep_first = keep;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.cap_log2 = softcap > 0.f ? softcap * 1.4426950408889634f : 0.f; a.scale_over_cap = softcap > 0.f ? scale / softcap : 0.f;
  a.r1 = r1; a.r2 = r2; a.sink = sink; a.v_row = v_row > 0 ? v_row : dv; a.n_splits = n_splits; a.part_o = part_o; a.part_ml = part_ml;
  a.dist_bias = dist_bias; a.dist_rows = dist_bias ? dist_rows : 1; a.gate_off = gate_off;
  cudaStream_t s = (cudaStream_t)stream;
#define BIASED_CASE(K, V) \
  if (dk == K && dv == V) return dist_bias ? biased_mma_launch<K, V, 2>(a, n_tiles, n_items, tiles, items, s) \
                                 : gate_off >= 0 ? biased_mma_launch<K, V, 1>(a, n_tiles, n_items, tiles, items, s) \
                                                 : biased_mma_launch<K, V, 0>(a, n_tiles, n_items, tiles, items, s);
  BIASED_SIZES(BIASED_CASE)
#undef BIASED_CASE
  return (int)cudaErrorInvalidValue;
}
