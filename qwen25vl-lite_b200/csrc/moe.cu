// Kernels of the routed feed-forward (a mixture of small gated feed-forwards, of which each token
// uses `top`):
//
//   z = Wr h (float), s = sigmoid(z); the `top` experts with the largest scores, weights s (as they are)
//   expert e on input a = s_e * h:  g = min(Wg a, limit), u = clamp(Wu a, -limit, limit),
//                                   y = Wd (g * sigmoid(alpha g) * (u + 1))
//   out = sum over the chosen experts of y  (+ sigmoid(Wsg h) * shared(h), the caller's product)
//
// The (token, expert) pairs of a step are sorted by expert on the device: the router counts, a
// one-block kernel lays the experts' rows out one after the other (each expert's rows filled up to
// a whole number of row tiles), a scatter kernel gives every pair its row.  Two grouped products
// then walk the row tiles, each tile belonging to one expert: gate and up with the activation in
// the epilogue, and down.  A last kernel adds a token's rows up in the order of its choices.
// Nothing is read back by the host, so a step can be captured into a graph; the grids are sized
// for the most tiles there can be and the tiles past the count leave at once.
//
// Every output element of the plain products is one FMA chain over k in order, whatever tile the
// row falls into, so a token's result does not depend on the batch.  The bfloat16 products run on
// the tensor cores (mma.sync m16n8k16, float accumulators) with the same layout.
#include "attention_decode.cuh"
#include "row_logits.cuh"

#define MOE_MAX_EXPERTS ROW_LOGITS_MAX
#define MOE_MAX_TOP 16

// One block of 8 warps per TOK tokens (4 in steps of many tokens, where a row of the router read from
// cache then serves four tokens; 1 otherwise): the tokens' rows are widened to float in shared memory
// once; each warp takes every eighth expert (and in its turn the shared expert's gate) and forms the
// logits with the lanes striding over the channels four at a time, then a butterfly: an order that
// depends on the sizes alone, whatever the step.  Then a warp per token picks the `top` largest
// (ties to the lower index).
template <typename T, int TOK>
__global__ void __launch_bounds__(256)
moe_route_kernel(const T* __restrict__ h, const float* __restrict__ router, const float* __restrict__ shared_gate,
                 int* __restrict__ topk_idx, float* __restrict__ topk_w, float* __restrict__ sg,
                 int* __restrict__ counts, int n_tokens, int hidden, int experts, int top) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) float route_smem[];       // TOK rows of hidden floats, then TOK x (MOE_MAX_EXPERTS + 1) logits
  route_logits<T, TOK>(h, router, shared_gate, route_smem, n_tokens, hidden, experts);
  const int pitch = (hidden + 3) & ~3;
  float* zs = route_smem + TOK * pitch;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * TOK;
  if (warp >= TOK || n0 + warp >= n_tokens) return;
  const int n = n0 + warp;
  float* z_row = zs + warp * (MOE_MAX_EXPERTS + 1);
  if (shared_gate && lane == 0) sg[n] = 1.0f / (1.0f + expf(-z_row[experts]));
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float z = z_row[e];
      if (z > best) { best = z; arg = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
    }
    if (lane == 0) {
      topk_idx[(size_t)n * top + k] = arg;
      topk_w[(size_t)n * top + k] = 1.0f / (1.0f + expf(-best));
      z_row[arg] = -INFINITY;
      atomicAdd(&counts[arg], 1);
    }
    __syncwarp();
  }
}

// The router of a mixture whose scores are a softmax over all `outputs` router rows, the last `outputs - experts` of
// which stand for experts without matrices (a choice among them takes no row of the grouped products).  The choice looks
// at score + correction[e]; the rows form `groups` equal runs of neighbours, a run's mark is its largest such number, and
// only the `keep` runs with the largest marks can be chosen from (the others count as minus infinity).  The `top`
// largest are chosen (ties to the lower index, among runs too); a choice weighs in with its plain score: as it is, or
// with renorm divided by the sum of the token's chosen scores (+ 1e-20); either way times weight_scale.  counts: one per
// expert with matrices.  One block of 8 warps per TOK tokens as above, then a warp per token.
template <typename T, int TOK>
__global__ void __launch_bounds__(256)
moe_route_softmax_kernel(const T* __restrict__ h, const float* __restrict__ router, const float* __restrict__ correction,
                         int* __restrict__ topk_idx, float* __restrict__ topk_w, int* __restrict__ counts, int n_tokens, int hidden,
                         int experts, int outputs, int top, int groups, int keep, int renorm, float weight_scale) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) float route_smem[];       // TOK rows of hidden floats, then TOK x 3 x (MOE_MAX_EXPERTS + 1) numbers
  route_logits<T, TOK>(h, router, nullptr, route_smem, n_tokens, hidden, outputs);
  const int pitch = (hidden + 3) & ~3;
  float* zs = route_smem + TOK * pitch;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * TOK;
  if (warp >= TOK || n0 + warp >= n_tokens) return;
  const int n = n0 + warp;
  float* score = zs + warp * (MOE_MAX_EXPERTS + 1);                          // logits, then scores
  float* choice = zs + (TOK + 2 * warp) * (MOE_MAX_EXPERTS + 1);             // score + correction
  float* mark = choice + (MOE_MAX_EXPERTS + 1);                              // a run's mark
  float top_z = -INFINITY;
  for (int e = lane; e < outputs; e += 32) top_z = fmaxf(top_z, score[e]);
  top_z = warp_max(top_z);
  float sum = 0.f;
  for (int e = lane; e < outputs; e += 32) { const float p = expf(score[e] - top_z); score[e] = p; sum += p; }
  sum = warp_sum(sum);
  __syncwarp();
  for (int e = lane; e < outputs; e += 32) {
    const float s = score[e] / sum;
    score[e] = s;
    choice[e] = s + (correction ? correction[e] : 0.f);
  }
  __syncwarp();
  if (groups > 1) {
    const int per = outputs / groups;
    for (int g = lane; g < groups; g += 32) {
      float best = -INFINITY;
      for (int e = g * per; e < (g + 1) * per; ++e) best = fmaxf(best, choice[e]);
      mark[g] = best;
    }
    __syncwarp();
    // the kept runs one after the other; every lane holds the same set: bit g % 32 of word g / 32
    unsigned kept[MOE_MAX_EXPERTS / 32];
#pragma unroll
    for (int i = 0; i < MOE_MAX_EXPERTS / 32; ++i) kept[i] = 0u;
    for (int k = 0; k < keep; ++k) {
      float best = -INFINITY;
      int arg = 0x7fffffff;
      for (int g = lane; g < groups; g += 32) {
        bool taken = false;
#pragma unroll
        for (int i = 0; i < MOE_MAX_EXPERTS / 32; ++i) if (i == (g >> 5)) taken = (kept[i] >> (g & 31)) & 1u;
        const float v = mark[g];
        if (!taken && v > best) { best = v; arg = g; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
        if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
      }
      if (arg != 0x7fffffff) {
#pragma unroll
        for (int i = 0; i < MOE_MAX_EXPERTS / 32; ++i) if (i == (arg >> 5)) kept[i] |= 1u << (arg & 31);
      }
    }
    for (int e = lane; e < outputs; e += 32) {
      const int g = e / per;
      bool ok = false;
#pragma unroll
      for (int i = 0; i < MOE_MAX_EXPERTS / 32; ++i) if (i == (g >> 5)) ok = (kept[i] >> (g & 31)) & 1u;
      if (!ok) choice[e] = -INFINITY;
    }
    __syncwarp();
  }
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int e = lane; e < outputs; e += 32) {
      const float c = choice[e];
      if (c > best) { best = c; arg = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
    }
    if (lane == 0) {
      // fewer choosable rows than `top` (the host refuses such sizes): the choice is row 0 with weight 0
      const bool none = arg == 0x7fffffff;
      topk_idx[(size_t)n * top + k] = none ? 0 : arg;
      mark[k] = none ? 0.f : score[arg];                        // the marks of the runs have served: the chosen scores wait here
      if (!none) {
        choice[arg] = -INFINITY;
        if (arg < experts) atomicAdd(&counts[arg], 1);
      } else {
        atomicAdd(&counts[0], 1);
      }
    }
    __syncwarp();
  }
  float chosen = 0.f;                                           // in the order of the choices, the same in every lane
  if (renorm) for (int k = 0; k < top; ++k) chosen += mark[k];
  for (int k = lane; k < top; k += 32) topk_w[(size_t)n * top + k] = (renorm ? mark[k] / (chosen + 1e-20f) : mark[k]) * weight_scale;
}

// One block: where every expert's rows begin (each expert filled up to whole tiles of `tile` rows),
// which expert every tile belongs to, how many tiles there are; all rows marked empty.
// plan: [0] number of tiles, [1 .. experts+1] first row of each expert (and the end), then the tiles' experts.
__global__ void moe_plan_kernel(const int* __restrict__ counts, int* __restrict__ plan, int* __restrict__ row_pair,
                                int experts, int tile, int max_rows) {
  pdl_trigger();
  pdl_wait();
  if (threadIdx.x == 0) {
    int row = 0, t = 0;
    int* first = plan + 1;
    int* tile_expert = plan + 2 + experts;
    for (int e = 0; e < experts; ++e) {
      first[e] = row;
      const int tiles = (counts[e] + tile - 1) / tile;
      for (int i = 0; i < tiles; ++i) tile_expert[t++] = e;
      row += tiles * tile;
    }
    first[experts] = row;
    plan[0] = t;
  }
  for (int r = threadIdx.x; r < max_rows; r += blockDim.x) row_pair[r] = -1;
}

__global__ void moe_scatter_kernel(const int* __restrict__ topk_idx, const int* __restrict__ plan, int* __restrict__ cursor,
                                   int* __restrict__ row_pair, int* __restrict__ pair_row, int n_pairs, int experts) {
  pdl_trigger();
  pdl_wait();
  const int pair = blockIdx.x * blockDim.x + threadIdx.x;
  if (pair >= n_pairs) return;
  const int e = topk_idx[pair];
  if (e >= experts) { pair_row[pair] = -1; return; }      // a choice beyond the experts that have matrices takes no row
  const int r = plan[1 + e] + atomicAdd(&cursor[e], 1);
  row_pair[r] = pair;
  pair_row[pair] = r;
}

// Grouped product on the CUDA cores.  GATE_UP: rows are the tile's pairs, a = weight * h[token];
// two chains per element (gate, up), activation in the epilogue, out = act [rows, N] in T.
// Otherwise: rows are act rows, one chain, out = y [rows, N] in float.  W* are [experts, N, K].
template <typename T, bool GATE_UP, int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
moe_grouped_fma_kernel(const T* __restrict__ A, const T* __restrict__ W0, const T* __restrict__ W1, void* __restrict__ out_,
                       const int* __restrict__ plan, const int* __restrict__ row_pair, const float* __restrict__ topk_w,
                       int experts, int top, int N, int K, long long w_stride, float limit, float alpha, float shift) {
  pdl_trigger();
  pdl_wait();
  constexpr int THREADS = (BM / TM) * (BN / TN);
  const int tile = blockIdx.y;
  if (tile >= plan[0]) return;
  const int e = plan[2 + experts + tile];
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws0[BK][BN + 4];
  __shared__ float Ws1[GATE_UP ? BK : 1][BN + 4];
  __shared__ int src_row[BM];
  __shared__ float src_w[BM];
  const int m0 = tile * BM, n0 = blockIdx.x * BN;
  for (int r = threadIdx.x; r < BM; r += THREADS) {
    const int pair = row_pair[m0 + r];
    if (GATE_UP) {
      src_row[r] = pair < 0 ? -1 : pair / top;
      src_w[r] = pair < 0 ? 0.f : (topk_w ? topk_w[pair] : 1.f);      // no weights: the rows as they are
    } else {
      src_row[r] = pair < 0 ? -1 : m0 + r;
      src_w[r] = 1.f;
    }
  }
  __syncthreads();
  const int tx = threadIdx.x % (BN / TN), ty = threadIdx.x / (BN / TN);
  const T* w0 = W0 + (size_t)e * w_stride;              // w_stride: values from one expert's matrix to the next one's
  const T* w1 = GATE_UP ? W1 + (size_t)e * w_stride : nullptr;
  float acc0[TM][TN], acc1[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc0[i][j] = acc1[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int x = threadIdx.x; x < BM * BK; x += THREADS) {
      const int r = x / BK, c = x % BK;
      const int gk = k0 + c, src = src_row[r];
      float v = 0.f;
      if (src >= 0 && gk < K) v = to_f32(A[(size_t)src * K + gk]);
      As[c][r] = GATE_UP ? v * src_w[r] : v;
    }
    for (int x = threadIdx.x; x < BN * BK; x += THREADS) {
      const int r = x / BK, c = x % BK;
      const int gn = n0 + r, gk = k0 + c;
      const bool ok = gn < N && gk < K;
      Ws0[c][r] = ok ? to_f32(w0[(size_t)gn * K + gk]) : 0.f;
      if (GATE_UP) Ws1[c][r] = ok ? to_f32(w1[(size_t)gn * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b0[TN], b1[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) {
        b0[j] = Ws0[kk][tx * TN + j];
        if (GATE_UP) b1[j] = Ws1[kk][tx * TN + j];
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          acc0[i][j] = fmaf(a[i], b0[j], acc0[i][j]);
          if (GATE_UP) acc1[i][j] = fmaf(a[i], b1[j], acc1[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int r = ty * TM + i;
    if (src_row[r] < 0) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx * TN + j;
      if (gn >= N) continue;
      if (GATE_UP) {
        const float g = fminf(acc0[i][j], limit);
        const float u = fminf(fmaxf(acc1[i][j], -limit), limit);
        reinterpret_cast<T*>(out_)[(size_t)(m0 + r) * N + gn] = from_f32<T>(g / (1.0f + expf(-alpha * g)) * (u + shift));
      } else {
        reinterpret_cast<float*>(out_)[(size_t)(m0 + r) * N + gn] = acc0[i][j];
      }
    }
  }
}

// The rows of the sorted pairs as the tensor-core product reads them: sorted[row, :] = weight of
// the pair * h[token of the pair, :], rounded to bfloat16.  One block per row; empty rows are left
// as they are (their products are never stored).
__global__ void moe_gather_kernel(const bf16* __restrict__ h, const int* __restrict__ row_pair, const float* __restrict__ topk_w,
                                  bf16* __restrict__ sorted, int top, int K) {
  pdl_trigger();
  pdl_wait();
  const int pair = row_pair[blockIdx.x];
  if (pair < 0) return;
  const float w = topk_w ? topk_w[pair] : 1.f;
  const bf16* src = h + (size_t)(pair / top) * K;
  bf16* dst = sorted + (size_t)blockIdx.x * K;
  for (int c = threadIdx.x * 8; c < K; c += blockDim.x * 8) {
    uint4 v = *reinterpret_cast<const uint4*>(src + c);
    unsigned* u = reinterpret_cast<unsigned*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 x = *reinterpret_cast<__nv_bfloat162*>(&u[i]);
      u[i] = pack_bf16(__low2float(x) * w, __high2float(x) * w);
    }
    *reinterpret_cast<uint4*>(dst + c) = v;
  }
}

// The grouped products on the tensor cores (bfloat16, mma.sync m16n8k16, float accumulators): a CTA
// of 4 warps takes a tile of BM rows x 64 columns of one expert.  BM = 16 (steps of few rows: a
// stream of the experts' weights): the warps split the columns, 16 each.  BM = 64: 2 x 2 warps of
// 32 rows x 32 columns.  BM = 128: the warps split the rows, 32 rows x 64 columns each, so that a
// fragment of the weights read from shared memory feeds two products and a fragment of A eight
// (sixteen with gate and up).  A is [rows, K], the rows in the sorted order.  K is walked in
// steps of 64 through a ring of STAGES stages filled by 16-byte cp.async (the rows of A and of the
// weights alike), so that a CTA always has several stages in flight.  Every element's sum runs over
// K in the same order whatever tile the row is in.
template <bool GATE_UP, int BM, int WARPS_M, int STAGES>
__global__ void __launch_bounds__(128)
moe_grouped_mma_kernel(const bf16* __restrict__ A, const bf16* __restrict__ W0, const bf16* __restrict__ W1, void* __restrict__ out_,
                       const int* __restrict__ plan, const int* __restrict__ row_pair, int experts, int N, int K, long long w_stride,
                       float limit, float alpha, float shift) {
  pdl_trigger();
  pdl_wait();
  constexpr int BN = 64, BK = 64, P = BK * 2 + 16;            // pitch in bytes: an odd number of 16-byte chunks
  constexpr int WARPS_N = 4 / WARPS_M, WM = BM / WARPS_M, WN = BN / WARPS_N;
  constexpr int MI = WM / 16, NJ = WN / 8;
  static_assert(WM % 16 == 0 && NJ % 2 == 0, "a warp holds whole 16-row blocks and pairs of 8-column blocks");
  constexpr int A_BYTES = BM * P, W_BYTES = BN * P, STAGE = A_BYTES + (GATE_UP ? 2 : 1) * W_BYTES;
  const int tile = blockIdx.y;
  if (tile >= plan[0]) return;
  const int e = plan[2 + experts + tile];
  extern __shared__ __align__(16) unsigned char ring[];
  __shared__ int src_row[BM];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int m0 = tile * BM, n0 = blockIdx.x * BN;
  for (int r = threadIdx.x; r < BM; r += 128) src_row[r] = row_pair[m0 + r];
  const bf16* w0 = W0 + (size_t)e * w_stride;
  const bf16* w1 = GATE_UP ? W1 + (size_t)e * w_stride : nullptr;
  const bf16* a0 = A + (size_t)m0 * K;
  const int nk = (K + BK - 1) / BK;
  auto load = [&](int kt) {
    unsigned char* st = ring + (kt % STAGES) * STAGE;
    const int k0 = kt * BK;
    for (int x = threadIdx.x; x < (BM + BN) * (BK / 8); x += 128) {
      const int r = x / (BK / 8), ch = x % (BK / 8);
      const int gk = k0 + ch * 8;
      if (r < BM) {
        cp_async16(st + r * P + ch * 16, a0 + (gk < K ? (size_t)r * K + gk : 0), gk < K);
      } else {
        const int gn = n0 + r - BM;
        const bool ok = gn < N && gk < K;
        const size_t off = ok ? (size_t)gn * K + gk : 0;
        cp_async16(st + A_BYTES + (r - BM) * P + ch * 16, w0 + off, ok);
        if (GATE_UP) cp_async16(st + A_BYTES + W_BYTES + (r - BM) * P + ch * 16, w1 + off, ok);
      }
    }
  };
  const int row_base = (warp / WARPS_N) * WM, col_base = (warp % WARPS_N) * WN;
  float acc0[MI][NJ][4], acc1[GATE_UP ? MI : 1][GATE_UP ? NJ : 1][4];
#pragma unroll
  for (int i = 0; i < MI; ++i)
#pragma unroll
    for (int j = 0; j < NJ; ++j) acc0[i][j][0] = acc0[i][j][1] = acc0[i][j][2] = acc0[i][j][3] = 0.f;
  if (GATE_UP) {
#pragma unroll
    for (int i = 0; i < MI; ++i)
#pragma unroll
      for (int j = 0; j < NJ; ++j) acc1[i][j][0] = acc1[i][j][1] = acc1[i][j][2] = acc1[i][j][3] = 0.f;
  }
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < nk) load(s);
    cp_async_commit();
  }
  for (int kt = 0; kt < nk; ++kt) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();                          // tile kt has landed, and everybody is done with tile kt - 1
    if (kt + STAGES - 1 < nk) load(kt + STAGES - 1);
    cp_async_commit();
    const unsigned char* st = ring + (kt % STAGES) * STAGE;
    const unsigned char* Ws0 = st + A_BYTES;
    const unsigned char* Ws1 = Ws0 + W_BYTES;
#pragma unroll
    for (int kk = 0; kk < BK / 16; ++kk) {
      // all fragments of the step first, then all its products: a product does not wait for the load just before it
      unsigned a[MI][4], b0[NJ / 2][4], b1[GATE_UP ? NJ / 2 : 1][4];
#pragma unroll
      for (int i = 0; i < MI; ++i) ldmatrix_x4(a[i], st + (row_base + i * 16 + (lane & 15)) * P + (kk * 16 + 8 * (lane >> 4)) * 2);
#pragma unroll
      for (int jp = 0; jp < NJ / 2; ++jp) {
        // two 8-column blocks at a time: (columns 0-7, k 0-7), (0-7, k 8-15), (8-15, k 0-7), (8-15, k 8-15)
        const int off = (col_base + jp * 16 + (lane & 7) + 8 * (lane >> 4)) * P + (kk * 16 + 8 * ((lane >> 3) & 1)) * 2;
        ldmatrix_x4(b0[jp], Ws0 + off);
        if (GATE_UP) ldmatrix_x4(b1[jp], Ws1 + off);
      }
#pragma unroll
      for (int jp = 0; jp < NJ / 2; ++jp) {
#pragma unroll
        for (int i = 0; i < MI; ++i) {
          mma_bf16(acc0[i][2 * jp], a[i], b0[jp][0], b0[jp][1]);
          mma_bf16(acc0[i][2 * jp + 1], a[i], b0[jp][2], b0[jp][3]);
        }
        if (GATE_UP) {
#pragma unroll
          for (int i = 0; i < MI; ++i) {
            mma_bf16(acc1[i][2 * jp], a[i], b1[jp][0], b1[jp][1]);
            mma_bf16(acc1[i][2 * jp + 1], a[i], b1[jp][2], b1[jp][3]);
          }
        }
      }
    }
  }
  cp_async_wait<0>();
#pragma unroll
  for (int i = 0; i < MI; ++i) {
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int r = row_base + i * 16 + g + 8 * half;
        if (src_row[r] < 0) continue;
        const int gn = n0 + col_base + j * 8 + 2 * t;
        if (gn >= N) continue;
        const float v0 = acc0[i][j][2 * half], v1 = acc0[i][j][2 * half + 1];
        if (GATE_UP) {
          const float g0 = fminf(v0, limit), g1 = fminf(v1, limit);
          const float u0 = fminf(fmaxf(acc1[i][j][2 * half], -limit), limit), u1 = fminf(fmaxf(acc1[i][j][2 * half + 1], -limit), limit);
          const float y0 = g0 / (1.0f + expf(-alpha * g0)) * (u0 + shift), y1 = g1 / (1.0f + expf(-alpha * g1)) * (u1 + shift);
          bf16* o = reinterpret_cast<bf16*>(out_) + (size_t)(m0 + r) * N + gn;
          if (gn + 1 < N && N % 2 == 0) *reinterpret_cast<unsigned*>(o) = pack_bf16(y0, y1);
          else { o[0] = __float2bfloat16_rn(y0); if (gn + 1 < N) o[1] = __float2bfloat16_rn(y1); }
        } else {
          float* o = reinterpret_cast<float*>(out_) + (size_t)(m0 + r) * N + gn;
          o[0] = v0;
          if (gn + 1 < N) o[1] = v1;
        }
      }
    }
  }
}

// out[n, :] = sum over the token's choices, in their order, of y[row of the pair, :]
//             (+ sg[n] * shared[n, :]), in T.
template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ pair_row, const float* __restrict__ sg,
                                   const T* __restrict__ shared, T* __restrict__ out, int n_tokens, int hidden, int top) {
  pdl_trigger();
  pdl_wait();
  // a block per token: its rows are looked up once; four channels at a time where the width allows
  const int n = blockIdx.x;
  __shared__ int rows[MOE_MAX_TOP];
  if (threadIdx.x < top) rows[threadIdx.x] = pair_row[(size_t)n * top + threadIdx.x];
  __syncthreads();
  const float gate = shared ? sg[n] : 0.f;
  if (hidden % 4 == 0 && !(((uintptr_t)y | (uintptr_t)shared | (uintptr_t)out) & 15)) {
    for (int c = threadIdx.x * 4; c < hidden; c += blockDim.x * 4) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int k = 0; k < top; ++k) {
        const float4 v = *reinterpret_cast<const float4*>(y + (size_t)rows[k] * hidden + c);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      if (shared) {
        float s4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) s4[i] = to_f32(shared[(size_t)n * hidden + c + i]);
        acc.x = fmaf(gate, s4[0], acc.x); acc.y = fmaf(gate, s4[1], acc.y); acc.z = fmaf(gate, s4[2], acc.z); acc.w = fmaf(gate, s4[3], acc.w);
      }
      T* o = out + (size_t)n * hidden + c;
      o[0] = from_f32<T>(acc.x); o[1] = from_f32<T>(acc.y); o[2] = from_f32<T>(acc.z); o[3] = from_f32<T>(acc.w);
    }
  } else {
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      float acc = 0.f;
      for (int k = 0; k < top; ++k) acc += y[(size_t)rows[k] * hidden + c];
      if (shared) acc = fmaf(gate, to_f32(shared[(size_t)n * hidden + c]), acc);
      out[(size_t)n * hidden + c] = from_f32<T>(acc);
    }
  }
}

// out[n, :] = sum over the token's choices, in their order, of w[pair] * (y[row of the pair, :], or the token's own
// input h[n, :] when the pair has no row: a choice that stands for an expert without matrices), plus shared[n, :] when
// given (an expert that every token uses, unweighted), in T.
template <typename T>
__global__ void moe_combine_weighted_kernel(const float* __restrict__ y, const int* __restrict__ pair_row, const float* __restrict__ topk_w,
                                            const T* __restrict__ h, const T* __restrict__ shared, T* __restrict__ out, int n_tokens,
                                            int hidden, int top) {
  pdl_trigger();
  pdl_wait();
  const int n = blockIdx.x;
  __shared__ int rows[MOE_MAX_TOP];
  __shared__ float ws[MOE_MAX_TOP];
  if (threadIdx.x < top) {
    rows[threadIdx.x] = pair_row[(size_t)n * top + threadIdx.x];
    ws[threadIdx.x] = topk_w[(size_t)n * top + threadIdx.x];
  }
  __syncthreads();
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k) {
      const float v = rows[k] >= 0 ? y[(size_t)rows[k] * hidden + c] : to_f32(h[(size_t)n * hidden + c]);
      acc = fmaf(ws[k], v, acc);
    }
    if (shared) acc += to_f32(shared[(size_t)n * hidden + c]);
    out[(size_t)n * hidden + c] = from_f32<T>(acc);
  }
}

// Rows that the sorted pairs can take at most: every pair, and each expert filled up to a tile.
Q25_EXPORT int q25_moe_max_rows(int n_pairs, int experts, int tile) {
  const int most_tiles = (n_pairs + tile - 1) / tile + experts;
  return most_tiles * tile;
}

template <typename T, int TOK>
static int moe_route_shape(const void* h, const float* router, const float* shared_gate, int* topk_idx, float* topk_w, float* sg,
                           int* counts, int n_tokens, int hidden, int experts, int top, cudaStream_t stream) {
  const size_t smem = (size_t)TOK * (((hidden + 3) & ~3) + MOE_MAX_EXPERTS + 1) * sizeof(float);
  if (smem > 200 * 1024) return -1;
  if (smem > 48 * 1024) {
    const cudaError_t e = cudaFuncSetAttribute(moe_route_kernel<T, TOK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  launch(moe_route_kernel<T, TOK>, dim3((n_tokens + TOK - 1) / TOK), dim3(256), smem, stream, (const T*)h, router, shared_gate, topk_idx,
         topk_w, sg, counts, n_tokens, hidden, experts, top);
  return launch_status();
}

template <typename T>
static int moe_route(const void* h, const float* router, const float* shared_gate, int* topk_idx, float* topk_w, float* sg,
                     int* counts, int n_tokens, int hidden, int experts, int top, void* stream) {
  if (n_tokens <= 0) return 0;
  if (experts <= 0 || experts > MOE_MAX_EXPERTS || top <= 0 || top > experts || top > MOE_MAX_TOP) return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  int rc = -1;
  if (n_tokens >= 512) rc = moe_route_shape<T, 4>(h, router, shared_gate, topk_idx, topk_w, sg, counts, n_tokens, hidden, experts, top, s);
  if (rc == -1) rc = moe_route_shape<T, 1>(h, router, shared_gate, topk_idx, topk_w, sg, counts, n_tokens, hidden, experts, top, s);
  return rc == -1 ? (int)cudaErrorInvalidValue : rc;
}

Q25_EXPORT int q25_moe_route_f32(const void* h, const float* r, const float* g, int* ti, float* tw, float* sg, int* counts, int n,
                                 int hidden, int experts, int top, void* s) {
  return moe_route<float>(h, r, g, ti, tw, sg, counts, n, hidden, experts, top, s);
}
Q25_EXPORT int q25_moe_route_bf16(const void* h, const float* r, const float* g, int* ti, float* tw, float* sg, int* counts, int n,
                                  int hidden, int experts, int top, void* s) {
  return moe_route<bf16>(h, r, g, ti, tw, sg, counts, n, hidden, experts, top, s);
}

// counts and cursor: `experts` ints each, zero on entry (cursor is left as the counts).
Q25_EXPORT int q25_moe_sort(const int* topk_idx, const int* counts, int* cursor, int* plan, int* row_pair, int* pair_row, int n_pairs,
                            int experts, int tile, void* stream) {
  if (n_pairs <= 0) return 0;
  const int max_rows = q25_moe_max_rows(n_pairs, experts, tile);
  launch(moe_plan_kernel, dim3(1), dim3(256), 0, (cudaStream_t)stream, counts, plan, row_pair, experts, tile, max_rows);
  launch(moe_scatter_kernel, dim3((n_pairs + 255) / 256), dim3(256), 0, (cudaStream_t)stream, topk_idx, (const int*)plan, cursor, row_pair,
         pair_row, n_pairs, experts);
  return launch_status();
}

template <bool GATE_UP, int BM, int WARPS_M, int STAGES>
static int moe_grouped_mma_shape(const void* A, const void* W0, const void* W1, void* out, const int* plan, const int* row_pair,
                                 int tiles, int experts, int N, int K, long long w_stride, float limit, float alpha, float shift, cudaStream_t s) {
  constexpr int SMEM = STAGES * (BM + (GATE_UP ? 128 : 64)) * (64 * 2 + 16);
  const cudaError_t e = cudaFuncSetAttribute(moe_grouped_mma_kernel<GATE_UP, BM, WARPS_M, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
  if (e != cudaSuccess) return (int)e;
  launch(moe_grouped_mma_kernel<GATE_UP, BM, WARPS_M, STAGES>, dim3((N + 63) / 64, tiles), dim3(128), SMEM, s, (const bf16*)A, (const bf16*)W0,
         (const bf16*)W1, out, plan, row_pair, experts, N, K, w_stride, limit, alpha, shift);
  return launch_status();
}

// A: the rows in the sorted order, [rows, K] bfloat16.
template <bool GATE_UP>
static int moe_grouped_mma(const void* A, const void* W0, const void* W1, void* out, const int* plan, const int* row_pair,
                           int n_pairs, int experts, int N, int K, long long w_stride, float limit, float alpha, float shift, int tile, void* stream) {
  const int tiles = q25_moe_max_rows(n_pairs, experts, tile) / tile;
  cudaStream_t s = (cudaStream_t)stream;
  if (tile == 16) return moe_grouped_mma_shape<GATE_UP, 16, 1, 4>(A, W0, W1, out, plan, row_pair, tiles, experts, N, K, w_stride, limit, alpha, shift, s);
  // two stages for the large tiles: three or four CTAs then share an SM (12 to 16 warps), which hides the fixed latencies between
  // a fragment's load and its products better than a third stage does (gate and up at 4,096 rows: 268 us with three stages)
  if (tile == 64) return moe_grouped_mma_shape<GATE_UP, 64, 2, 2>(A, W0, W1, out, plan, row_pair, tiles, experts, N, K, w_stride, limit, alpha, shift, s);
  if (tile == 128) return moe_grouped_mma_shape<GATE_UP, 128, 4, 2>(A, W0, W1, out, plan, row_pair, tiles, experts, N, K, w_stride, limit, alpha, shift, s);
  return (int)cudaErrorInvalidValue;
}

static bool moe_mma_takes(const void* A, const void* W0, const void* W1, const void* extra, int K) {
  return K % 8 == 0 && !(((uintptr_t)A | (uintptr_t)W0 | (uintptr_t)W1 | (uintptr_t)extra) & 15);
}

template <typename T, bool GATE_UP>
static int moe_grouped_fma(const void* A, const void* W0, const void* W1, void* out, const int* plan, const int* row_pair,
                           const float* topk_w, int n_pairs, int experts, int top, int N, int K, long long w_stride, float limit,
                           float alpha, float shift, int tile, void* stream) {
  if (n_pairs <= 0) return 0;
  const int tiles = q25_moe_max_rows(n_pairs, experts, tile) / tile;
  if (tile == 16) {
    launch(moe_grouped_fma_kernel<T, GATE_UP, 16, 64, 16, 1, 4>, dim3((N + 63) / 64, tiles), dim3(256), 0, (cudaStream_t)stream,
           (const T*)A, (const T*)W0, (const T*)W1, out, plan, row_pair, topk_w, experts, top, N, K, w_stride, limit, alpha, shift);
  } else if (tile == 64) {
    launch(moe_grouped_fma_kernel<T, GATE_UP, 64, 64, 16, 4, 4>, dim3((N + 63) / 64, tiles), dim3(256), 0, (cudaStream_t)stream,
           (const T*)A, (const T*)W0, (const T*)W1, out, plan, row_pair, topk_w, experts, top, N, K, w_stride, limit, alpha, shift);
  } else if (tile == 128) {     // the rows were laid out for the tensor-core product, which then did not take the operands
    launch(moe_grouped_fma_kernel<T, GATE_UP, 128, 64, 16, 8, 4>, dim3((N + 63) / 64, tiles), dim3(256), 0, (cudaStream_t)stream,
           (const T*)A, (const T*)W0, (const T*)W1, out, plan, row_pair, topk_w, experts, top, N, K, w_stride, limit, alpha, shift);
  } else {
    return (int)cudaErrorInvalidValue;
  }
  return launch_status();
}

// wgu: the experts' gate and up matrices, [experts, 2 * ff, hidden]: an expert's ff gate rows, then its
// ff up rows.  sorted: [max rows, hidden] of scratch in the activation dtype for the rows in the sorted
// order (bfloat16: the tensor-core product reads them; nullptr or float: the product gathers by itself).
Q25_EXPORT int q25_moe_gate_up_f32(const void* h, const void* wgu, void* act, const int* plan, const int* row_pair,
                                   const float* topk_w, int n_pairs, int experts, int top, int ff, int hidden, float limit,
                                   float alpha, float shift, int tile, void* sorted, void* s) {
  const float* w = (const float*)wgu;
  return moe_grouped_fma<float, true>(h, w, w + (size_t)ff * hidden, act, plan, row_pair, topk_w, n_pairs, experts, top, ff, hidden,
                                      2LL * ff * hidden, limit, alpha, shift, tile, s);
}
Q25_EXPORT int q25_moe_gather_bf16(const void* h, const int* row_pair, const float* topk_w, void* sorted, int rows, int top, int hidden,
                                   void* s) {
  if (rows <= 0) return 0;
  if (hidden % 8 || (((uintptr_t)h | (uintptr_t)sorted) & 15)) return (int)cudaErrorInvalidValue;
  launch(moe_gather_kernel, dim3(rows), dim3(128), 0, (cudaStream_t)s, (const bf16*)h, row_pair, topk_w, (bf16*)sorted, top, hidden);
  return launch_status();
}
Q25_EXPORT int q25_moe_gate_up_bf16(const void* h, const void* wgu, void* act, const int* plan, const int* row_pair,
                                    const float* topk_w, int n_pairs, int experts, int top, int ff, int hidden, float limit,
                                    float alpha, float shift, int tile, void* sorted, void* s) {
  if (n_pairs <= 0) return 0;
  const bf16* w = (const bf16*)wgu;
  const bf16* wu = w + (size_t)ff * hidden;
  if (sorted && moe_mma_takes(h, w, wu, sorted, hidden)) {
    launch(moe_gather_kernel, dim3(q25_moe_max_rows(n_pairs, experts, tile)), dim3(128), 0, (cudaStream_t)s, (const bf16*)h, row_pair, topk_w,
           (bf16*)sorted, top, hidden);
    return moe_grouped_mma<true>(sorted, w, wu, act, plan, row_pair, n_pairs, experts, ff, hidden, 2LL * ff * hidden, limit, alpha, shift, tile, s);
  }
  return moe_grouped_fma<bf16, true>(h, w, wu, act, plan, row_pair, topk_w, n_pairs, experts, top, ff, hidden, 2LL * ff * hidden, limit, alpha, shift,
                                     tile, s);
}
Q25_EXPORT int q25_moe_down_f32(const void* act, const void* wd, void* y, const int* plan, const int* row_pair, int n_pairs,
                                int experts, int top, int hidden, int ff, int tile, void* s) {
  return moe_grouped_fma<float, false>(act, wd, nullptr, y, plan, row_pair, nullptr, n_pairs, experts, top, hidden, ff, (long long)hidden * ff,
                                       0.f, 0.f, 0.f, tile, s);
}
Q25_EXPORT int q25_moe_down_bf16(const void* act, const void* wd, void* y, const int* plan, const int* row_pair, int n_pairs,
                                 int experts, int top, int hidden, int ff, int tile, void* s) {
  if (n_pairs <= 0) return 0;
  if (moe_mma_takes(act, wd, nullptr, nullptr, ff))
    return moe_grouped_mma<false>(act, wd, nullptr, y, plan, row_pair, n_pairs, experts, hidden, ff, (long long)hidden * ff, 0.f, 0.f, 0.f, tile, s);
  return moe_grouped_fma<bf16, false>(act, wd, nullptr, y, plan, row_pair, nullptr, n_pairs, experts, top, hidden, ff, (long long)hidden * ff,
                                      0.f, 0.f, 0.f, tile, s);
}

template <typename T>
static int moe_combine(const float* y, const int* pair_row, const float* sg, const void* shared, void* out, int n_tokens, int hidden,
                       int top, void* stream) {
  if (n_tokens <= 0) return 0;
  launch(moe_combine_kernel<T>, dim3(n_tokens), dim3(hidden >= 2048 ? 256 : 128), 0, (cudaStream_t)stream, y, pair_row, sg,
         (const T*)shared, (T*)out, n_tokens, hidden, top);
  return launch_status();
}
Q25_EXPORT int q25_moe_combine_f32(const float* y, const int* pr, const float* sg, const void* sh, void* out, int n, int h, int top, void* s) {
  return moe_combine<float>(y, pr, sg, sh, out, n, h, top, s);
}
Q25_EXPORT int q25_moe_combine_bf16(const float* y, const int* pr, const float* sg, const void* sh, void* out, int n, int h, int top, void* s) {
  return moe_combine<bf16>(y, pr, sg, sh, out, n, h, top, s);
}

template <typename T, int TOK>
static int moe_route_softmax_shape(const void* h, const float* router, const float* correction, int* topk_idx, float* topk_w, int* counts,
                                   int n_tokens, int hidden, int experts, int outputs, int top, int groups, int keep, int renorm,
                                   float weight_scale, cudaStream_t stream) {
  const size_t smem = (size_t)TOK * (((hidden + 3) & ~3) + 3 * (MOE_MAX_EXPERTS + 1)) * sizeof(float);
  if (smem > 200 * 1024) return -1;
  if (smem > 48 * 1024) {
    const cudaError_t e = cudaFuncSetAttribute(moe_route_softmax_kernel<T, TOK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  launch(moe_route_softmax_kernel<T, TOK>, dim3((n_tokens + TOK - 1) / TOK), dim3(256), smem, stream, (const T*)h, router, correction,
         topk_idx, topk_w, counts, n_tokens, hidden, experts, outputs, top, groups, keep, renorm, weight_scale);
  return launch_status();
}

template <typename T>
static int moe_route_softmax(const void* h, const float* router, const float* correction, int* topk_idx, float* topk_w, int* counts,
                             int n_tokens, int hidden, int experts, int outputs, int top, int groups, int keep, int renorm,
                             float weight_scale, void* stream) {
  if (n_tokens <= 0) return 0;
  if (experts <= 0 || outputs < experts || outputs > MOE_MAX_EXPERTS || top <= 0 || top > MOE_MAX_TOP || groups < 1 || outputs % groups ||
      keep < 1 || keep > groups || top > keep * (outputs / groups))
    return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  int rc = -1;
  if (n_tokens >= 512) rc = moe_route_softmax_shape<T, 4>(h, router, correction, topk_idx, topk_w, counts, n_tokens, hidden, experts, outputs, top, groups, keep, renorm, weight_scale, s);
  if (rc == -1) rc = moe_route_softmax_shape<T, 1>(h, router, correction, topk_idx, topk_w, counts, n_tokens, hidden, experts, outputs, top, groups, keep, renorm, weight_scale, s);
  return rc == -1 ? (int)cudaErrorInvalidValue : rc;
}
Q25_EXPORT int q25_moe_route_softmax_f32(const void* h, const float* r, const float* corr, int* ti, float* tw, int* counts, int n, int hidden,
                                         int experts, int outputs, int top, int groups, int keep, int renorm, float wscale, void* s) {
  return moe_route_softmax<float>(h, r, corr, ti, tw, counts, n, hidden, experts, outputs, top, groups, keep, renorm, wscale, s);
}
Q25_EXPORT int q25_moe_route_softmax_bf16(const void* h, const float* r, const float* corr, int* ti, float* tw, int* counts, int n, int hidden,
                                          int experts, int outputs, int top, int groups, int keep, int renorm, float wscale, void* s) {
  return moe_route_softmax<bf16>(h, r, corr, ti, tw, counts, n, hidden, experts, outputs, top, groups, keep, renorm, wscale, s);
}

template <typename T>
static int moe_combine_weighted(const float* y, const int* pair_row, const float* topk_w, const void* h, const void* shared, void* out,
                                int n_tokens, int hidden, int top, void* stream) {
  if (n_tokens <= 0) return 0;
  if (top > MOE_MAX_TOP) return (int)cudaErrorInvalidValue;
  launch(moe_combine_weighted_kernel<T>, dim3(n_tokens), dim3(hidden >= 2048 ? 256 : 128), 0, (cudaStream_t)stream, y, pair_row, topk_w,
         (const T*)h, (const T*)shared, (T*)out, n_tokens, hidden, top);
  return launch_status();
}
Q25_EXPORT int q25_moe_combine_weighted_f32(const float* y, const int* pr, const float* tw, const void* h, const void* sh, void* out, int n, int hd, int top, void* s) {
  return moe_combine_weighted<float>(y, pr, tw, h, sh, out, n, hd, top, s);
}
Q25_EXPORT int q25_moe_combine_weighted_bf16(const float* y, const int* pr, const float* tw, const void* h, const void* sh, void* out, int n, int hd, int top, void* s) {
  return moe_combine_weighted<bf16>(y, pr, tw, h, sh, out, n, hd, top, s);
}
