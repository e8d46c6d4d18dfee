// Embedding gather (alone, or with a learned position vector and the model's norm), fused
// residual-add + RMSNorm (plain, or in groups with an update that is normalised on its way in),
// SiLU-mul, clamped gated linear unit.
//
// Formulas (reference: zhangjianbang-nb/qwen25vl-lite):
//   embedding   x[n,:] = E[token[n],:]                          src/qwen25vl_lite/text.py:213
//   RMSNorm     h = x * rsqrt(mean(x^2) + eps) * w              src/qwen25vl_lite/layers.py:27-31
//   SwiGLU act  f = silu(g) * u, silu(z) = z / (1 + exp(-z))    src/qwen25vl_lite/text.py:66
// The residual stream x is float in both dtypes; the norm fuses the pending residual update
// (x += delta) so that a block's output is read once.
#include "common.cuh"

template <typename T>
__global__ void embed_gather_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ x, int hidden, int vocab, float scale) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  int id = ids[row];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);  // the host validates ids; never read outside
  const T* src = table + (size_t)id * hidden;
  float* dst = x + (size_t)row * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = to_f32(src[c]) * scale;      // scale 1: the row as it is
}

// Four consecutive values as floats, and back (bf16: 8 bytes, float: 16 bytes at a time).
template <typename T> __device__ __forceinline__ float4 load4(const T* p);
template <> __device__ __forceinline__ float4 load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 load4<bf16>(const bf16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
template <typename T> __device__ __forceinline__ void store4(T* p, float4 v);
template <> __device__ __forceinline__ void store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void store4<bf16>(bf16* p, float4 v) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<const unsigned*>(&a);
  raw.y = *reinterpret_cast<const unsigned*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

// x[row] += delta[row] (if delta), then out[r] = rmsnorm(x[row]) * w.
// rows == nullptr: row = r, x is updated in place.  rows != nullptr: row = rows[r], x is left
// untouched (used for the final norm, which only the wanted positions need).
// VEC: hidden is a multiple of 4 and every row starts on a 16-byte boundary, so a thread moves four
// values at a time.  The sum of squares is taken thread by thread, then lanes, then warps, in a fixed
// order that depends on hidden alone.
template <typename T, bool EXACT, bool VEC>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const T* __restrict__ delta,
                                   const float* __restrict__ w, float eps, T* __restrict__ out,
                                   const int* __restrict__ rows, int hidden) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) float row_cache[];  // hidden floats + 32 scratch
  float* scratch = row_cache + hidden;
  const int r = blockIdx.x;
  const int row = rows ? rows[r] : r;
  float* xr = x + (size_t)row * hidden;
  const T* dr = delta ? delta + (size_t)row * hidden : nullptr;
  T* o = out + (size_t)r * hidden;
  float ss = 0.f;
  if (VEC) {
    for (int c = threadIdx.x * 4; c < hidden; c += blockDim.x * 4) {
      float4 v = *reinterpret_cast<const float4*>(xr + c);
      if (dr) {
        const float4 d = load4<T>(dr + c);
        v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
        if (!rows) *reinterpret_cast<float4*>(xr + c) = v;
      }
      *reinterpret_cast<float4*>(row_cache + c) = v;
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  } else {
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      float v = xr[c];
      if (dr) {
        v += to_f32(dr[c]);
        if (!rows) xr[c] = v;
      }
      row_cache[c] = v;
      ss += v * v;
    }
  }
  const float total = block_sum(ss, scratch);
  const float inv = EXACT ? 1.0f / sqrtf(total / (float)hidden + eps) : rsqrtf(total / (float)hidden + eps);
  if (VEC) {
    for (int c = threadIdx.x * 4; c < hidden; c += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(row_cache + c), ww = *reinterpret_cast<const float4*>(w + c);
      store4<T>(o + c, make_float4(v.x * inv * ww.x, v.y * inv * ww.y, v.z * inv * ww.z, v.w * inv * ww.w));
    }
  } else {
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) o[c] = from_f32<T>(row_cache[c] * inv * w[c]);
  }
}

// gu is [n, 2*inter].  paired == 0: gate in the first half of a row, up in the second.
// paired == 1: groups of 16 columns hold 8 gate features followed by their 8 up features (the
// layout the skinny GEMM's SwiGLU epilogue wants of the weight rows).
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int n, int inter, int paired) {
  pdl_trigger();
  pdl_wait();
  const size_t total = (size_t)n * inter;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t row = i / inter, c = i % inter;
    const size_t gc = paired ? (c >> 3) * 16 + (c & 7) : c;
    const size_t uc = paired ? gc + 8 : inter + c;
    const float g = to_f32(gu[row * 2 * inter + gc]);
    const float u = to_f32(gu[row * 2 * inter + uc]);
    out[i] = from_f32<T>(g / (1.0f + expf(-g)) * u);
  }
}

// ---- normalisation in groups ------------------------------------------------------------------------
// A row of `hidden` values is cut into `groups` equal consecutive parts and each part is divided by
// its own root mean square: v / sqrt(mean(part^2) + eps).  groups == 1 is the plain RMS norm.  The
// squares of a part are summed thread by thread, then lanes, then warps, in an order that depends on
// the sizes alone.  `inv` (shared, `groups` floats) receives 1 / rms of every part.
template <bool EXACT>
__device__ __forceinline__ void group_inverse_rms(const float* row_cache, int hidden, int groups, float eps, float* inv,
                                                  float* scratch) {
  // Each warp takes every (number of warps)-th group: its lanes stride over the group's values, four at
  // a time where the group's width allows, then a butterfly.  One barrier before (the row is in
  // shared memory) and one after (every group's figure is there), however many groups there are.
  const int width = hidden / groups;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  __syncthreads();
  for (int g = warp; g < groups; g += nwarps) {
    const float* part = row_cache + g * width;
    float ss = 0.f;
    if (width % 4 == 0 && hidden % 4 == 0) {
      for (int c = lane * 4; c < width; c += 128) {
        const float4 v = *reinterpret_cast<const float4*>(part + c);
        ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
      }
    } else {
      for (int c = lane; c < width; c += 32) ss = fmaf(part[c], part[c], ss);
    }
    ss = warp_sum(ss);
    if (lane == 0) inv[g] = EXACT ? 1.0f / sqrtf(ss / (float)width + eps) : rsqrtf(ss / (float)width + eps);
  }
  __syncthreads();
  (void)scratch;
}

#define NORM_MAX_GROUPS 64

// x[n,:] = norm_in_groups(E[token[n],:] * scale + P[position[n],:]) * w: a token embedding with a learned
// vector per position (not scaled) added before the model's norm; w == nullptr: no norm, the sum as it
// is.  The float32 residual stream starts here.
template <typename T, bool EXACT>
__global__ void embed_position_norm_kernel(const T* __restrict__ table, const T* __restrict__ pos_table,
                                           const int* __restrict__ ids, const int* __restrict__ positions,
                                           const float* __restrict__ w, float eps, float* __restrict__ x, int hidden,
                                           int vocab, int max_positions, int groups, float scale) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) float row_cache[];  // hidden floats + 32 scratch + groups
  float* scratch = row_cache + hidden;
  float* inv = scratch + 32;
  const int row = blockIdx.x;
  int id = ids[row], p = positions[row];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);                      // the host validates both; never read outside
  p = p < 0 ? 0 : (p >= max_positions ? max_positions - 1 : p);
  const T* e = table + (size_t)id * hidden;
  const T* q = pos_table + (size_t)p * hidden;
  float* dst0 = x + (size_t)row * hidden;
  if (!w) {
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst0[c] = fmaf(to_f32(e[c]), scale, to_f32(q[c]));
    return;
  }
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) row_cache[c] = fmaf(to_f32(e[c]), scale, to_f32(q[c]));
  __syncthreads();
  group_inverse_rms<EXACT>(row_cache, hidden, groups, eps, inv, scratch);
  const int width = hidden / groups;
  float* dst = x + (size_t)row * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = row_cache[c] * inv[c / width] * w[c];
}

// x[row] += d, where d = delta[row] as it is (dw == nullptr) or norm_in_groups(delta[row]) * dw (a
// sublayer that is normalised after as well as before); then out[r] = norm_in_groups(x[row]) * w.
// rows as in add_rmsnorm_kernel: with rows the sum is formed for those rows only and x is left alone.
// out == nullptr: only the addition.  w == nullptr: out[r] = x[row] as it is, in T (a sublayer that reads
// the stream itself).
template <typename T, bool EXACT, bool VEC>
__global__ void add_norm_groups_kernel(float* __restrict__ x, const T* __restrict__ delta, const float* __restrict__ dw,
                                       float d_eps, int d_groups, const float* __restrict__ w, float eps, int groups,
                                       T* __restrict__ out, const int* __restrict__ rows, int hidden) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) float row_cache[];  // 2 * hidden floats + 32 scratch + 2 * groups
  float* d_cache = row_cache + hidden;
  float* scratch = d_cache + hidden;
  float* inv = scratch + 32;
  float* d_inv = inv + NORM_MAX_GROUPS;
  const int r = blockIdx.x;
  const int row = rows ? rows[r] : r;
  float* xr = x + (size_t)row * hidden;
  constexpr int STEP = VEC ? 4 : 1;
  if (delta) {
    const T* dr = delta + (size_t)row * hidden;
    if (dw) {
      for (int c = threadIdx.x * STEP; c < hidden; c += blockDim.x * STEP) {
        if (VEC) *reinterpret_cast<float4*>(d_cache + c) = load4<T>(dr + c);
        else d_cache[c] = to_f32(dr[c]);
      }
      group_inverse_rms<EXACT>(d_cache, hidden, d_groups, d_eps, d_inv, scratch);
    }
    const int dwidth = dw ? hidden / d_groups : hidden;
    for (int c = threadIdx.x * STEP; c < hidden; c += blockDim.x * STEP) {
      if (VEC) {
        float4 v = *reinterpret_cast<const float4*>(xr + c);
        if (dw) {
          const float4 d = *reinterpret_cast<const float4*>(d_cache + c), ww = *reinterpret_cast<const float4*>(dw + c);
          const float s = d_inv[c / dwidth];
          v.x += d.x * s * ww.x; v.y += d.y * s * ww.y; v.z += d.z * s * ww.z; v.w += d.w * s * ww.w;
        } else {
          const float4 d = load4<T>(dr + c);
          v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
        }
        *reinterpret_cast<float4*>(row_cache + c) = v;
        if (!rows) *reinterpret_cast<float4*>(xr + c) = v;
      } else {
        const float v = xr[c] + (dw ? d_cache[c] * d_inv[c / dwidth] * dw[c] : to_f32(dr[c]));
        row_cache[c] = v;
        if (!rows) xr[c] = v;
      }
    }
  } else {
    for (int c = threadIdx.x * STEP; c < hidden; c += blockDim.x * STEP) {
      if (VEC) *reinterpret_cast<float4*>(row_cache + c) = *reinterpret_cast<const float4*>(xr + c);
      else row_cache[c] = xr[c];
    }
  }
  if (!out) return;
  T* o = out + (size_t)r * hidden;
  if (!w) {            // every thread reads back what it wrote itself
    for (int c = threadIdx.x * STEP; c < hidden; c += blockDim.x * STEP) {
      if (VEC) store4<T>(o + c, *reinterpret_cast<const float4*>(row_cache + c));
      else o[c] = from_f32<T>(row_cache[c]);
    }
    return;
  }
  group_inverse_rms<EXACT>(row_cache, hidden, groups, eps, inv, scratch);
  const int width = hidden / groups;
  for (int c = threadIdx.x * STEP; c < hidden; c += blockDim.x * STEP) {
    if (VEC) {
      const float4 v = *reinterpret_cast<const float4*>(row_cache + c), ww = *reinterpret_cast<const float4*>(w + c);
      const float s = inv[c / width];
      store4<T>(o + c, make_float4(v.x * s * ww.x, v.y * s * ww.y, v.z * s * ww.z, v.w * s * ww.w));
    } else {
      o[c] = from_f32<T>(row_cache[c] * inv[c / width] * w[c]);
    }
  }
}

// Gated linear unit with clamped branches: gu is [n, 2*inter], gate in the first half of a row, up
// in the second; g = min(g, limit), u = clamp(u, -limit, limit), out = g * sigmoid(alpha * g) * (u + shift)
// (limit infinite, alpha 1 and shift 0: silu(g) * u).
template <typename T, bool VEC>
__global__ void glu_clamped_kernel(const T* __restrict__ gu, T* __restrict__ out, int n, int inter, float limit, float alpha,
                                   float shift, int paired) {
  pdl_trigger();
  pdl_wait();
  constexpr int STEP = VEC ? 4 : 1;                     // VEC: inter is a multiple of 4 and the rows start on 16-byte boundaries
  const size_t total = (size_t)n * inter / STEP;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t row = i * STEP / inter, c = i * STEP % inter;
    // paired: groups of 8 gate features followed by their 8 up features (a run of 4 stays inside a group)
    const T* g_at = gu + row * 2 * inter + (paired ? (c >> 3) * 16 + (c & 7) : c);
    const size_t up_at = paired ? 8 : inter;
    float g[4], u[4];
    if (VEC) {
      const float4 gv = load4<T>(g_at), uv = load4<T>(g_at + up_at);
      g[0] = gv.x; g[1] = gv.y; g[2] = gv.z; g[3] = gv.w;
      u[0] = uv.x; u[1] = uv.y; u[2] = uv.z; u[3] = uv.w;
    } else {
      g[0] = to_f32(g_at[0]);
      u[0] = to_f32(g_at[up_at]);
    }
#pragma unroll
    for (int k = 0; k < STEP; ++k) {
      const float gg = fminf(g[k], limit), uu = fminf(fmaxf(u[k], -limit), limit);
      g[k] = gg / (1.0f + expf(-alpha * gg)) * (uu + shift);
    }
    if (VEC) store4<T>(out + i * 4, make_float4(g[0], g[1], g[2], g[3]));
    else out[i] = from_f32<T>(g[0]);
  }
}

// Dynamic Tanh, a norm without statistics: x[row] += delta[row] (when given), then
// out[r] = tanh(alpha * x[row]) * w + b.  rows as in add_rmsnorm_kernel: with rows only those rows
// are produced and x is left alone.  Nothing is reduced, so a row is just a run of elements.
template <typename T, bool VEC>
__global__ void add_dyt_kernel(float* __restrict__ x, const T* __restrict__ delta, const float* __restrict__ w,
                               const float* __restrict__ b, float alpha, T* __restrict__ out, const int* __restrict__ rows,
                               int hidden) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int row = rows ? rows[r] : r;
  float* xr = x + (size_t)row * hidden;
  const T* dr = delta ? delta + (size_t)row * hidden : nullptr;
  T* o = out + (size_t)r * hidden;
  if (VEC) {                                    // hidden is a multiple of 4 and every row starts on a 16-byte boundary
    for (int c = threadIdx.x * 4; c < hidden; c += blockDim.x * 4) {
      float4 v = *reinterpret_cast<const float4*>(xr + c);
      if (dr) {
        const float4 d = load4<T>(dr + c);
        v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
        if (!rows) *reinterpret_cast<float4*>(xr + c) = v;
      }
      const float4 ww = *reinterpret_cast<const float4*>(w + c), bb = *reinterpret_cast<const float4*>(b + c);
      store4<T>(o + c, make_float4(fmaf(tanhf(alpha * v.x), ww.x, bb.x), fmaf(tanhf(alpha * v.y), ww.y, bb.y),
                                   fmaf(tanhf(alpha * v.z), ww.z, bb.z), fmaf(tanhf(alpha * v.w), ww.w, bb.w)));
    }
  } else {
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      float v = xr[c];
      if (dr) {
        v += to_f32(dr[c]);
        if (!rows) xr[c] = v;
      }
      o[c] = from_f32<T>(fmaf(tanhf(alpha * v), w[c], b[c]));
    }
  }
}

// logits <- cap * tanh(logits / cap), in place.
__global__ void softcap_kernel(float* __restrict__ logits, size_t total, float cap) {
  pdl_trigger();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    logits[i] = cap * tanhf(logits[i] / cap);
}

template <typename T, bool EXACT>
static int embed_position_norm(const void* table, const void* pos_table, const int* ids, const int* positions, const float* w,
                               float eps, float* x, int n, int hidden, int vocab, int max_positions, int groups, float scale, void* stream) {
  if (n <= 0) return 0;
  if (groups <= 0 || groups > NORM_MAX_GROUPS || hidden % groups) return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)(hidden + 32 + NORM_MAX_GROUPS) * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  if (smem > 48 * 1024) {
    const cudaError_t e = cudaFuncSetAttribute(embed_position_norm_kernel<T, EXACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  launch(embed_position_norm_kernel<T, EXACT>, dim3(n), dim3(hidden >= 1024 ? 256 : 128), smem, (cudaStream_t)stream,
         (const T*)table, (const T*)pos_table, ids, positions, w, eps, x, hidden, vocab, max_positions, groups, scale);
  return launch_status();
}

template <typename T, bool EXACT>
static int add_norm_groups(float* x, const void* delta, const float* dw, float d_eps, int d_groups, const float* w, float eps,
                           int groups, void* out, const int* rows, int n_out, int hidden, void* stream) {
  if (n_out <= 0) return 0;
  if (groups <= 0 || groups > NORM_MAX_GROUPS || hidden % groups) return (int)cudaErrorInvalidValue;
  if (dw && (d_groups <= 0 || d_groups > NORM_MAX_GROUPS || hidden % d_groups)) return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)(2 * hidden + 32 + 2 * NORM_MAX_GROUPS) * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(add_norm_groups_kernel<T, EXACT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(add_norm_groups_kernel<T, EXACT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  // four values at a time when every group (of the stream's norm and of the update's) is a multiple of
  // four wide and every row starts on a 16-byte boundary
  const bool vec = hidden % 4 == 0 && (hidden / groups) % 4 == 0 && (!dw || (hidden / d_groups) % 4 == 0) &&
                   !(((uintptr_t)x | (uintptr_t)delta | (uintptr_t)dw | (uintptr_t)w | (uintptr_t)out) & 15);
  const dim3 block(hidden >= 1024 ? 256 : 128);
  if (vec) launch(add_norm_groups_kernel<T, EXACT, true>, dim3(n_out), block, smem, (cudaStream_t)stream, x, (const T*)delta, dw, d_eps,
                  d_groups, w, eps, groups, (T*)out, rows, hidden);
  else launch(add_norm_groups_kernel<T, EXACT, false>, dim3(n_out), block, smem, (cudaStream_t)stream, x, (const T*)delta, dw, d_eps,
              d_groups, w, eps, groups, (T*)out, rows, hidden);
  return launch_status();
}

template <typename T>
static int glu_clamped(const void* gu, void* out, int n, int inter, float limit, float alpha, float shift, int paired, void* stream) {
  if (n <= 0) return 0;
  if (paired && inter % 8) return (int)cudaErrorInvalidValue;
  const bool vec = inter % 4 == 0 && !(((uintptr_t)gu | (uintptr_t)out) & 15);
  const size_t total = (size_t)n * inter / (vec ? 4 : 1);
  size_t blocks = (total + 255) / 256;
  const size_t most = (size_t)(device_sm_count() > 0 ? device_sm_count() : 148) * 16;
  if (blocks > most) blocks = most;
  if (vec) launch(glu_clamped_kernel<T, true>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (const T*)gu, (T*)out, n, inter, limit, alpha, shift, paired);
  else launch(glu_clamped_kernel<T, false>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (const T*)gu, (T*)out, n, inter, limit, alpha, shift, paired);
  return launch_status();
}

template <typename T>
static int embed_gather(const void* table, const int* ids, float* x, int n, int hidden, int vocab, float scale, void* stream) {
  if (n <= 0) return 0;
  launch(embed_gather_kernel<T>, dim3(n), dim3(256), 0, (cudaStream_t)stream, (const T*)table, ids, x, hidden, vocab, scale);
  return launch_status();
}

template <typename T, bool EXACT>
static int add_rmsnorm(float* x, const void* delta, const float* w, float eps, void* out, const int* rows,
                       int n_out, int hidden, void* stream) {
  if (n_out <= 0) return 0;
  const size_t smem = (size_t)(hidden + 32) * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_kernel<T, EXACT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(add_rmsnorm_kernel<T, EXACT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int threads = hidden >= 1024 ? 256 : 128;
  const bool vec = hidden % 4 == 0 && !(((uintptr_t)x | (uintptr_t)delta | (uintptr_t)w | (uintptr_t)out) & 15);
  if (vec) launch(add_rmsnorm_kernel<T, EXACT, true>, dim3(n_out), dim3(threads), smem, (cudaStream_t)stream, x, (const T*)delta, w, eps, (T*)out, rows, hidden);
  else launch(add_rmsnorm_kernel<T, EXACT, false>, dim3(n_out), dim3(threads), smem, (cudaStream_t)stream, x, (const T*)delta, w, eps, (T*)out, rows, hidden);
  return launch_status();
}

template <typename T>
static int silu_mul(const void* gu, void* out, int n, int inter, int paired, void* stream) {
  if (n <= 0) return 0;
  const size_t total = (size_t)n * inter;
  size_t blocks = (total + 255) / 256;
  const size_t most = (size_t)(device_sm_count() > 0 ? device_sm_count() : 148) * 16;
  if (blocks > most) blocks = most;
  launch(silu_mul_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (const T*)gu, (T*)out, n, inter, paired);
  return launch_status();
}

Q25_EXPORT int q25_embed_gather_f32(const void* t, const int* ids, float* x, int n, int h, int v, float sc, void* s) { return embed_gather<float>(t, ids, x, n, h, v, sc, s); }
Q25_EXPORT int q25_embed_gather_bf16(const void* t, const int* ids, float* x, int n, int h, int v, float sc, void* s) { return embed_gather<bf16>(t, ids, x, n, h, v, sc, s); }
Q25_EXPORT int q25_add_rmsnorm_f32(float* x, const void* d, const float* w, float eps, void* o, const int* rows, int n, int h, void* s) { return add_rmsnorm<float, true>(x, d, w, eps, o, rows, n, h, s); }
Q25_EXPORT int q25_add_rmsnorm_bf16(float* x, const void* d, const float* w, float eps, void* o, const int* rows, int n, int h, void* s) { return add_rmsnorm<bf16, false>(x, d, w, eps, o, rows, n, h, s); }
Q25_EXPORT int q25_silu_mul_f32(const void* gu, void* o, int n, int inter, int paired, void* s) { return silu_mul<float>(gu, o, n, inter, paired, s); }
Q25_EXPORT int q25_silu_mul_bf16(const void* gu, void* o, int n, int inter, int paired, void* s) { return silu_mul<bf16>(gu, o, n, inter, paired, s); }

Q25_EXPORT int q25_embed_position_norm_f32(const void* t, const void* pt, const int* ids, const int* pos, const float* w, float eps, float* x, int n, int h, int v, int mp, int g, float sc, void* s) { return embed_position_norm<float, true>(t, pt, ids, pos, w, eps, x, n, h, v, mp, g, sc, s); }
Q25_EXPORT int q25_embed_position_norm_bf16(const void* t, const void* pt, const int* ids, const int* pos, const float* w, float eps, float* x, int n, int h, int v, int mp, int g, float sc, void* s) { return embed_position_norm<bf16, false>(t, pt, ids, pos, w, eps, x, n, h, v, mp, g, sc, s); }
Q25_EXPORT int q25_add_norm_groups_f32(float* x, const void* d, const float* dw, float de, int dg, const float* w, float eps, int g, void* o, const int* rows, int n, int h, void* s) { return add_norm_groups<float, true>(x, d, dw, de, dg, w, eps, g, o, rows, n, h, s); }
Q25_EXPORT int q25_add_norm_groups_bf16(float* x, const void* d, const float* dw, float de, int dg, const float* w, float eps, int g, void* o, const int* rows, int n, int h, void* s) { return add_norm_groups<bf16, false>(x, d, dw, de, dg, w, eps, g, o, rows, n, h, s); }
Q25_EXPORT int q25_glu_clamped_f32(const void* gu, void* o, int n, int inter, float limit, float alpha, float shift, int paired, void* s) { return glu_clamped<float>(gu, o, n, inter, limit, alpha, shift, paired, s); }
Q25_EXPORT int q25_glu_clamped_bf16(const void* gu, void* o, int n, int inter, float limit, float alpha, float shift, int paired, void* s) { return glu_clamped<bf16>(gu, o, n, inter, limit, alpha, shift, paired, s); }

// Streaming multiprocessors of the current device (0 if it cannot be read).
Q25_EXPORT int q25_sm_count(void) { return device_sm_count(); }

template <typename T>
static int add_dyt(float* x, const void* delta, const float* w, const float* b, float alpha, void* out, const int* rows, int n_out,
                   int hidden, void* stream) {
  if (n_out <= 0) return 0;
  const bool vec = hidden % 4 == 0 && !(((uintptr_t)x | (uintptr_t)delta | (uintptr_t)w | (uintptr_t)b | (uintptr_t)out) & 15);
  const dim3 block(hidden >= 1024 ? 256 : 128);
  if (vec) launch(add_dyt_kernel<T, true>, dim3(n_out), block, 0, (cudaStream_t)stream, x, (const T*)delta, w, b, alpha, (T*)out, rows, hidden);
  else launch(add_dyt_kernel<T, false>, dim3(n_out), block, 0, (cudaStream_t)stream, x, (const T*)delta, w, b, alpha, (T*)out, rows, hidden);
  return launch_status();
}
Q25_EXPORT int q25_add_dyt_f32(float* x, const void* d, const float* w, const float* b, float alpha, void* o, const int* rows, int n, int h, void* s) { return add_dyt<float>(x, d, w, b, alpha, o, rows, n, h, s); }
Q25_EXPORT int q25_add_dyt_bf16(float* x, const void* d, const float* w, const float* b, float alpha, void* o, const int* rows, int n, int h, void* s) { return add_dyt<bf16>(x, d, w, b, alpha, o, rows, n, h, s); }
Q25_EXPORT int q25_softcap(float* logits, long long total, float cap, void* s) {
  if (total <= 0) return 0;
  size_t blocks = ((size_t)total + 255) / 256;
  const size_t most = (size_t)(device_sm_count() > 0 ? device_sm_count() : 148) * 16;
  if (blocks > most) blocks = most;
  launch(softcap_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)s, logits, (size_t)total, cap);
  return launch_status();
}

// ---- layer norm around the residual stream; several branches into one update; a stream that is mixed with another ----

// (v - mean) / sqrt(var + eps) over the `hidden` floats of `row` (shared memory), var the mean of the squared
// deviations: two passes, each a block sum in a fixed order.  Returns (mean, 1 / sqrt(var + eps)) to every thread.
// VEC: four channels at a time (hidden is a multiple of 4).
template <bool VEC>
__device__ __forceinline__ float2 row_mean_inv(const float* row, int hidden, float eps, float* scratch) {
  float s = 0.f;
  if (VEC) {
    for (int c = threadIdx.x * 4; c < hidden; c += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(row + c);
      s += (v.x + v.y) + (v.z + v.w);
    }
  } else {
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) s += row[c];
  }
  const float mean = block_sum(s, scratch) / (float)hidden;
  float q = 0.f;
  if (VEC) {
    for (int c = threadIdx.x * 4; c < hidden; c += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(row + c);
      const float d0 = v.x - mean, d1 = v.y - mean, d2 = v.z - mean, d3 = v.w - mean;
      q += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
    }
  } else {
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) { const float d = row[c] - mean; q = fmaf(d, d, q); }
  }
  const float var = block_sum(q, scratch) / (float)hidden;
  return make_float2(mean, 1.0f / sqrtf(var + eps));
}

// x += post(delta); out = ((x - mean) / sqrt(var + eps)) * w + b.  post(delta), when dw is given, is the layer norm of
// the update with weight dw and bias db, times the vector ds when that is given (a learned scale per channel); without dw
// the update is added as it is.  With `rows` only those rows are produced and x is left alone.  out == nullptr: only the addition.
template <typename T, bool VEC>
__global__ void add_layernorm_kernel(float* __restrict__ x, const T* __restrict__ delta, const float* __restrict__ dw,
                                     const float* __restrict__ db, const float* __restrict__ ds, float d_eps,
                                     const float* __restrict__ w, const float* __restrict__ b, float eps,
                                     T* __restrict__ out, const int* __restrict__ rows, int hidden) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) float ln_cache[];     // 2 * hidden floats + 32 scratch
  float* row_cache = ln_cache;
  float* d_cache = ln_cache + hidden;
  float* scratch = d_cache + hidden;
  const int r = blockIdx.x;
  const int row = rows ? rows[r] : r;
  float* xr = x + (size_t)row * hidden;
  constexpr int STEP = VEC ? 4 : 1;
  const int c0 = threadIdx.x * STEP, dc = blockDim.x * STEP;
  if (delta) {
    const T* dr = delta + (size_t)row * hidden;
    float2 st = make_float2(0.f, 1.f);
    if (dw) {
      for (int c = c0; c < hidden; c += dc) {
        if (VEC) *reinterpret_cast<float4*>(d_cache + c) = load4<T>(dr + c);
        else d_cache[c] = to_f32(dr[c]);
      }
      __syncthreads();
      st = row_mean_inv<VEC>(d_cache, hidden, d_eps, scratch);
    }
    for (int c = c0; c < hidden; c += dc) {
      if (VEC) {
        float4 d = dw ? *reinterpret_cast<const float4*>(d_cache + c) : load4<T>(dr + c);
        if (dw) {
          const float4 ww = *reinterpret_cast<const float4*>(dw + c), bb = *reinterpret_cast<const float4*>(db + c);
          d.x = (d.x - st.x) * st.y * ww.x + bb.x; d.y = (d.y - st.x) * st.y * ww.y + bb.y;
          d.z = (d.z - st.x) * st.y * ww.z + bb.z; d.w = (d.w - st.x) * st.y * ww.w + bb.w;
          if (ds) {
            const float4 ss = *reinterpret_cast<const float4*>(ds + c);
            d.x *= ss.x; d.y *= ss.y; d.z *= ss.z; d.w *= ss.w;
          }
        }
        float4 v = *reinterpret_cast<const float4*>(xr + c);
        v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
        *reinterpret_cast<float4*>(row_cache + c) = v;
        if (!rows) *reinterpret_cast<float4*>(xr + c) = v;
      } else {
        float d = dw ? d_cache[c] : to_f32(dr[c]);
        if (dw) {
          d = (d - st.x) * st.y * dw[c] + db[c];
          if (ds) d *= ds[c];
        }
        const float v = xr[c] + d;
        row_cache[c] = v;
        if (!rows) xr[c] = v;
      }
    }
  } else {
    for (int c = c0; c < hidden; c += dc) {
      if (VEC) *reinterpret_cast<float4*>(row_cache + c) = *reinterpret_cast<const float4*>(xr + c);
      else row_cache[c] = xr[c];
    }
  }
  if (!out) return;
  __syncthreads();
  const float2 st = row_mean_inv<VEC>(row_cache, hidden, eps, scratch);
  T* o = out + (size_t)r * hidden;
  for (int c = c0; c < hidden; c += dc) {
    if (VEC) {
      const float4 v = *reinterpret_cast<const float4*>(row_cache + c), ww = *reinterpret_cast<const float4*>(w + c),
                   bb = *reinterpret_cast<const float4*>(b + c);
      store4<T>(o + c, make_float4((v.x - st.x) * st.y * ww.x + bb.x, (v.y - st.x) * st.y * ww.y + bb.y, (v.z - st.x) * st.y * ww.z + bb.z,
                                   (v.w - st.x) * st.y * ww.w + bb.w));
    } else {
      o[c] = from_f32<T>((row_cache[c] - st.x) * st.y * w[c] + b[c]);
    }
  }
}

template <typename T, bool VEC>
static int add_layernorm_shape(float* x, const void* delta, const float* dw, const float* db, const float* ds, float d_eps, const float* w,
                               const float* b, float eps, void* out, const int* rows, int n_out, int hidden, size_t smem, void* stream) {
  if (smem > 48 * 1024) {
    const cudaError_t e = cudaFuncSetAttribute(add_layernorm_kernel<T, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  launch(add_layernorm_kernel<T, VEC>, dim3(n_out), dim3(hidden >= 1024 ? 256 : 128), smem, (cudaStream_t)stream, x, (const T*)delta, dw, db,
         ds, d_eps, w, b, eps, (T*)out, rows, hidden);
  return launch_status();
}

template <typename T>
static int add_layernorm(float* x, const void* delta, const float* dw, const float* db, const float* ds, float d_eps, const float* w,
                         const float* b, float eps, void* out, const int* rows, int n_out, int hidden, void* stream) {
  if (n_out <= 0) return 0;
  if (out && (!w || !b)) return (int)cudaErrorInvalidValue;
  if (dw && !db) return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)(2 * hidden + 32) * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  if (hidden % 8 == 0) return add_layernorm_shape<T, true>(x, delta, dw, db, ds, d_eps, w, b, eps, out, rows, n_out, hidden, smem, stream);
  return add_layernorm_shape<T, false>(x, delta, dw, db, ds, d_eps, w, b, eps, out, rows, n_out, hidden, smem, stream);
}
Q25_EXPORT int q25_add_layernorm_f32(float* x, const void* d, const float* dw, const float* db, const float* ds, float de, const float* w, const float* b, float eps, void* o, const int* rows, int n, int h, void* s) { return add_layernorm<float>(x, d, dw, db, ds, de, w, b, eps, o, rows, n, h, s); }
Q25_EXPORT int q25_add_layernorm_bf16(float* x, const void* d, const float* dw, const float* db, const float* ds, float de, const float* w, const float* b, float eps, void* o, const int* rows, int n, int h, void* s) { return add_layernorm<bf16>(x, d, dw, db, ds, de, w, b, eps, o, rows, n, h, s); }

// out = (1 / n) * sum over the n branches of  branch_i / rms(branch_i) * w_i  (rms with eps inside the root), n <= 4:
// the results of mixers that ran side by side on the same input become one update.
struct BranchArgs {
  const void* in[4];
  const float* w[4];
  int n;
};
template <typename T>
__global__ void branch_mean_norm_kernel(BranchArgs a, T* __restrict__ out, int hidden, float eps) {
  pdl_trigger();
  pdl_wait();
  __shared__ float scratch[32];
  const size_t base = (size_t)blockIdx.x * hidden;
  float inv[4];
  for (int i = 0; i < a.n; ++i) {
    const T* p = (const T*)a.in[i] + base;
    float q = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) { const float v = to_f32(p[c]); q = fmaf(v, v, q); }
    inv[i] = 1.0f / sqrtf(block_sum(q, scratch) / (float)hidden + eps);
  }
  const float share = 1.0f / (float)a.n;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float acc = 0.f;
    for (int i = 0; i < a.n; ++i) acc += to_f32(((const T*)a.in[i])[base + c]) * inv[i] * a.w[i][c];
    out[base + c] = from_f32<T>(acc * share);
  }
}
template <typename T>
static int branch_mean_norm(const void* const* in, const float* const* w, int n, void* out, int rows, int hidden, float eps, void* stream) {
  if (rows <= 0) return 0;
  if (n < 1 || n > 4) return (int)cudaErrorInvalidValue;
  BranchArgs a;
  for (int i = 0; i < 4; ++i) { a.in[i] = i < n ? in[i] : nullptr; a.w[i] = i < n ? w[i] : nullptr; }
  a.n = n;
  launch(branch_mean_norm_kernel<T>, dim3(rows), dim3(hidden >= 1024 ? 256 : 128), 0, (cudaStream_t)stream, a, (T*)out, hidden, eps);
  return launch_status();
}
Q25_EXPORT int q25_branch_mean_norm_f32(const void* const* in, const float* const* w, int n, void* o, int rows, int h, float eps, void* s) { return branch_mean_norm<float>(in, w, n, o, rows, h, eps, s); }
Q25_EXPORT int q25_branch_mean_norm_bf16(const void* const* in, const float* const* w, int n, void* o, int rows, int h, float eps, void* s) { return branch_mean_norm<bf16>(in, w, n, o, rows, h, eps, s); }

// cat[row] = [x[row] + post(delta)[row] | other[row]] in T, the input of a product that mixes the stream with another one
// (x itself is updated too: the pending update is in afterwards); and x = y + bias after that product:
template <typename T>
__global__ void stream_pair_kernel(const float* __restrict__ x, const float* __restrict__ other, T* __restrict__ cat, int hidden) {
  pdl_trigger();
  pdl_wait();
  const size_t row = blockIdx.x;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    cat[row * 2 * hidden + c] = from_f32<T>(x[row * hidden + c]);
    cat[row * 2 * hidden + hidden + c] = from_f32<T>(other[row * hidden + c]);
  }
}
__global__ void stream_set_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ bias, int hidden) {
  pdl_trigger();
  pdl_wait();
  const size_t row = blockIdx.x;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) x[row * hidden + c] = y[row * hidden + c] + bias[c];
}
Q25_EXPORT int q25_stream_pair_f32(const float* x, const float* other, void* cat, int rows, int h, void* s) {
  if (rows <= 0) return 0;
  launch(stream_pair_kernel<float>, dim3(rows), dim3(128), 0, (cudaStream_t)s, x, other, (float*)cat, h);
  return launch_status();
}
Q25_EXPORT int q25_stream_pair_bf16(const float* x, const float* other, void* cat, int rows, int h, void* s) {
  if (rows <= 0) return 0;
  launch(stream_pair_kernel<bf16>, dim3(rows), dim3(128), 0, (cudaStream_t)s, x, other, (bf16*)cat, h);
  return launch_status();
}
Q25_EXPORT int q25_stream_set(float* x, const float* y, const float* bias, int rows, int h, void* s) {
  if (rows <= 0) return 0;
  launch(stream_set_kernel, dim3(rows), dim3(128), 0, (cudaStream_t)s, x, y, bias, h);
  return launch_status();
}

// A feed-forward's activation on its own: out = act(in) element by element, in float.  kind 0: the square of
// relu, max(z, 0)^2; kind 1: gelu in its tanh form, 0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3))).
__device__ __forceinline__ float unary_act(float z, int kind) {
  if (kind == 0) { const float r = fmaxf(z, 0.f); return r * r; }
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * fmaf(0.044715f * z * z, z, z)));
}
template <typename T>
__global__ void activation_kernel(const T* __restrict__ in, T* __restrict__ out, size_t total, int kind) {
  pdl_trigger();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    out[i] = from_f32<T>(unary_act(to_f32(in[i]), kind));
}
template <typename T>
static int activation(const void* in, void* out, long long total, int kind, void* stream) {
  if (total <= 0) return 0;
  if (kind < 0 || kind > 1) return (int)cudaErrorInvalidValue;
  size_t blocks = ((size_t)total + 255) / 256;
  const size_t most = (size_t)(device_sm_count() > 0 ? device_sm_count() : 148) * 16;
  if (blocks > most) blocks = most;
  launch(activation_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (const T*)in, (T*)out, (size_t)total, kind);
  return launch_status();
}
Q25_EXPORT int q25_activation_f32(const void* in, void* out, long long total, int kind, void* s) { return activation<float>(in, out, total, kind, s); }
Q25_EXPORT int q25_activation_bf16(const void* in, void* out, long long total, int kind, void* s) { return activation<bf16>(in, out, total, kind, s); }
