// Mixture of experts: routing on the device and one grouped product for all experts.
//
// moe_route: per token, s_e = sigmoid(z_e), or softmax(z)_e over all experts; the `top` experts with the largest
//   s_e + correction_e (no correction: s_e) are chosen (ties: the lower index); their weights are s_e * scale.  One
//   warp per token, 32-bit.
// moe_align: the (token, choice) pairs of the step, numbered token * top + choice, are grouped by expert into tiles
//   of `tile` rows: sorted_rows[tile * tile_rows + i] is a pair's number or -1 (padding), tile_expert[tile] the
//   tile's expert or -1 (no such tile).  The host knows only the upper bound of the tile count.
// moe_linear: out[row] = act(W[expert of the row's tile] . in[row / rows_per_input]) for every row named by
//   sorted_rows.  W: [experts, N, K].  Two kernels: FFMA tiles for float32 (every output element is one chain of
//   fmaf over ascending k, so a row's result does not depend on the tile it landed in) and mma.sync tiles for
//   bfloat16 (below).
// moe_combine: resid[t] += sum_c weight[t, c] * y[t * top + c] (+ sigmoid(gate logit) * shared[t]), choices in the
//   order the router found them; with pair_pos, y is in the grouped order and pair p lies in row pair_pos[p].
// moe_gather: the grouped order's input rows made contiguous (for a product that fetches A tiles by TMA).
// gelu: the exact (erf) GELU, element by element.
#include "common.cuh"

TLLM_DEFINE_LAST_ERROR

namespace tllm {

__device__ __forceinline__ float gelu_erf(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752440f)); }

constexpr int ROUTE_PER_LANE = 16;   // experts per lane: at most 512 experts

__global__ void moe_route_kernel(const float* __restrict__ logits, int ld, int n_experts, const float* __restrict__ correction,
                                 float scale, int top, int* __restrict__ ids, float* __restrict__ weights, int n_tokens,
                                 int softmax) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= n_tokens) return;
  const int lane = threadIdx.x & 31;
  float s[ROUTE_PER_LANE], c[ROUTE_PER_LANE];
  float zmax = -INFINITY, zsum = 0.f;
  if (softmax) {   // scores over all experts: exp(z - max) / sum, the sum taken lane by lane and then across the warp
#pragma unroll
    for (int i = 0; i < ROUTE_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (e < n_experts) zmax = fmaxf(zmax, logits[(size_t)t * ld + e]);
    }
    zmax = warp_max(zmax);
#pragma unroll
    for (int i = 0; i < ROUTE_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      s[i] = e < n_experts ? expf(logits[(size_t)t * ld + e] - zmax) : 0.f;
      zsum += s[i];
    }
    zsum = 1.f / warp_sum(zsum);
  }
#pragma unroll
  for (int i = 0; i < ROUTE_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    if (e < n_experts) {
      s[i] = softmax ? s[i] * zsum : 1.f / (1.f + expf(-logits[(size_t)t * ld + e]));
      c[i] = correction ? s[i] + correction[e] : s[i];
    } else {
      s[i] = 0.f;
      c[i] = -INFINITY;
    }
  }
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    float bs = 0.f;
#pragma unroll
    for (int i = 0; i < ROUTE_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (e < n_experts && (c[i] > best)) { best = c[i]; bi = e; bs = s[i]; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      const float os = __shfl_xor_sync(0xffffffffu, bs, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; bs = os; }
    }
    if (lane == 0) {
      ids[(size_t)t * top + k] = bi;
      weights[(size_t)t * top + k] = bs * scale;
    }
#pragma unroll
    for (int i = 0; i < ROUTE_PER_LANE; ++i)
      if (lane + 32 * i == bi) c[i] = -INFINITY;
  }
}

// One CTA.  Shared: counts[n_experts], start[n_experts] (ints).
__global__ void moe_align_kernel(const int* __restrict__ ids, int n_pairs, int n_experts, int tile, int max_tiles,
                                 int* __restrict__ sorted_rows, int* __restrict__ tile_expert, int* __restrict__ pair_pos) {
  extern __shared__ int sh[];
  int* counts = sh;
  int* start = sh + n_experts;
  pdl_trigger();
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) counts[e] = 0;
  pdl_wait();
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) atomicAdd(&counts[ids[i]], 1);
  for (int i = threadIdx.x; i < max_tiles * tile; i += blockDim.x) sorted_rows[i] = -1;
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < n_experts; ++e) {
      start[e] = at * tile;
      const int nt = (counts[e] + tile - 1) / tile;
      for (int x = 0; x < nt; ++x) tile_expert[at + x] = e;
      at += nt;
      counts[e] = 0;
    }
    for (; at < max_tiles; ++at) tile_expert[at] = -1;
  }
  __syncthreads();
  // Pairs of one expert keep their order (by token, then choice) only up to the order of these atomics; a row's result
  // does not depend on where in its expert's tiles it lies.
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int e = ids[i];
    const int at = start[e] + atomicAdd(&counts[e], 1);
    sorted_rows[at] = i;
    if (pair_pos) pair_pos[i] = at;     // where the pair's row lies in the grouped order
  }
}

// The rows of a grouped order made contiguous: out[p] = in[sorted_rows[p] / rows_per_input], zeros for padding, so
// that a product that fetches its A tiles by TMA can take them (16-byte pieces; k a multiple of 8).
__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ in, int ld_in, const int* __restrict__ sorted_rows,
                                  const int* __restrict__ tile_expert, int tile, int rows_per_input,
                                  __nv_bfloat16* __restrict__ out, int k) {
  pdl_trigger();
  pdl_wait();
  const int p = blockIdx.x;
  if (tile_expert[p / tile] < 0) return;      // a tile that does not exist is never read
  const int src = sorted_rows[p];
  const uint4* from = reinterpret_cast<const uint4*>(in + (size_t)(src < 0 ? 0 : src / rows_per_input) * ld_in);
  uint4* to = reinterpret_cast<uint4*>(out + (size_t)p * k);
  for (int c = threadIdx.x; c < k / 8; c += blockDim.x) to[c] = src < 0 ? make_uint4(0, 0, 0, 0) : from[c];
}

// Tile of TM rows x 64 columns, k in slices of 16; 256 threads, each TM/16 rows x 4 columns.
template <typename T, typename TO, int TM, bool GELU>
__global__ void __launch_bounds__(256) moe_linear_kernel(const T* __restrict__ in, int ld_in, const T* __restrict__ w,
                                                         const int* __restrict__ sorted_rows,
                                                         const int* __restrict__ tile_expert, TO* __restrict__ out,
                                                         int n, int k, int rows_per_input) {
  constexpr int TN = 64, TK = 16, RM = TM / 16;
  __shared__ float sa[TK][TM + 1];
  __shared__ float sb[TK][TN + 1];
  __shared__ int srow[TM];
  pdl_trigger();
  pdl_wait();
  const int e = tile_expert[blockIdx.x];
  if (e < 0) return;
  const int n0 = blockIdx.y * TN;
  const int tid = threadIdx.x;
  if (tid < TM) srow[tid] = sorted_rows[(size_t)blockIdx.x * TM + tid];
  __syncthreads();
  const T* we = w + (size_t)e * n * k;
  const int tr = tid / 16, tc = tid % 16;   // rows tr * RM .., columns tc * 4 ..
  float acc[RM][4];
#pragma unroll
  for (int i = 0; i < RM; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < k; k0 += TK) {
    for (int idx = tid; idx < TM * TK; idx += 256) {
      const int m = idx / TK, kk = idx % TK;
      const int row = srow[m];
      sa[kk][m] = (row >= 0 && k0 + kk < k) ? to_f32(in[(size_t)(row / rows_per_input) * ld_in + k0 + kk]) : 0.f;
    }
    for (int idx = tid; idx < TN * TK; idx += 256) {
      const int c = idx / TK, kk = idx % TK;
      sb[kk][c] = (n0 + c < n && k0 + kk < k) ? to_f32(we[(size_t)(n0 + c) * k + k0 + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      float av[RM], bv[4];
#pragma unroll
      for (int i = 0; i < RM; ++i) av[i] = sa[kk][tr * RM + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = sb[kk][tc * 4 + j];
#pragma unroll
      for (int i = 0; i < RM; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < RM; ++i) {
    const int row = srow[tr * RM + i];
    if (row < 0) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = n0 + tc * 4 + j;
      if (c < n) out[(size_t)row * n + c] = from_f32<TO>(GELU ? gelu_erf(acc[i][j]) : acc[i][j]);
    }
  }
}

// ---- the grouped product on the tensor cores (bfloat16, mma.sync.m16n8k16, 32-bit sums)
// A CTA owns BM rows of one expert's tile and 128 output columns; k in slices of 32 through a three- or four-stage cp.async
// ring (rows of 80 bytes in shared memory: ldmatrix reads eight of them without a bank conflict).  Eight warps:
// 2 x 4 of 64 x 32 outputs for tiles of 128 rows, of 32 x 32 for tiles of 64 rows, 1 x 8 of 16 x 16 for tiles of 16
// rows (decode).  A rows are
// gathered by the tile's row list; rows of padding read nothing.  K and the row strides are multiples of 8.
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void ldsm4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float* c, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename TO, int BM, bool GELU>
__global__ void __launch_bounds__(256) moe_linear_mma_kernel(const __nv_bfloat16* __restrict__ in, int ld_in,
                                                             const __nv_bfloat16* __restrict__ w,
                                                             const int* __restrict__ sorted_rows,
                                                             const int* __restrict__ tile_expert, TO* __restrict__ out,
                                                             int n, int k, int rows_per_input) {
  constexpr int BN = 128, BK = 32, LDS = 40, STAGES = BM == 16 ? 4 : 3;
  constexpr int WM = BM >= 64 ? 2 : 1, WN = 8 / WM;           // warps along rows and columns
  constexpr int WTM = BM / WM, WTN = BN / WN;                 // a warp's outputs: 64 x 32, 32 x 32 or 16 x 16
  constexpr int MI = WTM / 16, NI = WTN / 8;
  constexpr int A_PER_THREAD = (BM * 4 + 255) / 256;          // 16-byte pieces of A per thread and stage
  extern __shared__ __align__(16) unsigned char moe_smem[];
  typedef __nv_bfloat16 (*TileA)[BM][LDS];
  typedef __nv_bfloat16 (*TileB)[BN][LDS];
  TileA sa = reinterpret_cast<TileA>(moe_smem);
  TileB sb = reinterpret_cast<TileB>(moe_smem + sizeof(__nv_bfloat16) * STAGES * BM * LDS);
  int* srow = reinterpret_cast<int*>(moe_smem + sizeof(__nv_bfloat16) * STAGES * (BM + BN) * LDS);
  pdl_trigger();
  pdl_wait();
  const int e = tile_expert[blockIdx.x];
  if (e < 0) return;
  const int n0 = blockIdx.y * BN;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < BM) srow[tid] = sorted_rows[(size_t)blockIdx.x * BM + tid];
  __syncthreads();
  const __nv_bfloat16* we = w + (size_t)e * n * k;
  // what this thread copies per stage: its 16-byte pieces of A (BM * 4 in all) and two of B
  const __nv_bfloat16* a_ptr[A_PER_THREAD];
  bool a_ok[A_PER_THREAD];
#pragma unroll
  for (int x = 0; x < A_PER_THREAD; ++x) {
    const int idx = tid + x * 256;
    const int src = idx < BM * 4 ? srow[idx >> 2] : -1;
    a_ok[x] = src >= 0;
    a_ptr[x] = in + (size_t)(src < 0 ? 0 : src / rows_per_input) * ld_in + (idx & 3) * 8;
  }
  const int nk = (k + BK - 1) / BK;
  auto load = [&](int stage, int kb) {
    const int k0 = kb * BK;
#pragma unroll
    for (int x = 0; x < A_PER_THREAD; ++x) {
      const int idx = tid + x * 256, c = (idx & 3) * 8;
      if (idx < BM * 4) {
        const bool ok = a_ok[x] && k0 + c < k;
        cp_async16(&sa[stage][idx >> 2][c], a_ptr[x] + (ok ? k0 : 0), ok);
      }
    }
#pragma unroll
    for (int x = 0; x < 2; ++x) {
      const int idx = tid + x * 256, r = idx >> 2, c = (idx & 3) * 8;
      const bool ok = n0 + r < n && k0 + c < k;
      cp_async16(&sb[stage][r][c], we + (size_t)(ok ? n0 + r : 0) * k + (ok ? k0 + c : 0), ok);
    }
  };
  float acc[MI][NI][4];
#pragma unroll
  for (int i = 0; i < MI; ++i)
#pragma unroll
    for (int j = 0; j < NI; ++j)
#pragma unroll
      for (int x = 0; x < 4; ++x) acc[i][j][x] = 0.f;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < nk) load(s, s);
    asm volatile("cp.async.commit_group;");
  }
  const int wm = warp / WN, wn = warp % WN;
  for (int kb = 0; kb < nk; ++kb) {
    asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2));
    __syncthreads();
    if (kb + STAGES - 1 < nk) load((kb + STAGES - 1) % STAGES, kb + STAGES - 1);
    asm volatile("cp.async.commit_group;");
    const int st = kb % STAGES;
#pragma unroll
    for (int kk = 0; kk < BK; kk += 16) {
      unsigned af[MI][4], bf[NI][2];
#pragma unroll
      for (int i = 0; i < MI; ++i)
        ldsm4(af[i][0], af[i][1], af[i][2], af[i][3], &sa[st][wm * WTM + i * 16 + (lane & 15)][kk + (lane >> 4) * 8]);
#pragma unroll
      for (int j = 0; j < NI; j += 2)
        ldsm4(bf[j][0], bf[j][1], bf[j + 1][0], bf[j + 1][1],
              &sb[st][wn * WTN + j * 8 + (lane & 7) + (lane >> 4) * 8][kk + ((lane >> 3) & 1) * 8]);
#pragma unroll
      for (int i = 0; i < MI; ++i)
#pragma unroll
        for (int j = 0; j < NI; ++j) mma_bf16(acc[i][j], af[i], bf[j][0], bf[j][1]);
    }
  }
  asm volatile("cp.async.wait_group 0;");
#pragma unroll
  for (int i = 0; i < MI; ++i)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int row = srow[wm * WTM + i * 16 + (lane >> 2) + half * 8];
      if (row < 0) continue;
#pragma unroll
      for (int j = 0; j < NI; ++j) {
        const int c = n0 + wn * WTN + j * 8 + (lane & 3) * 2;
        float v0 = acc[i][j][half * 2], v1 = acc[i][j][half * 2 + 1];
        if (GELU) { v0 = gelu_erf(v0); v1 = gelu_erf(v1); }
        if (c < n) out[(size_t)row * n + c] = from_f32<TO>(v0);
        if (c + 1 < n) out[(size_t)row * n + c + 1] = from_f32<TO>(v1);
      }
    }
}

__global__ void moe_combine_kernel(const float* __restrict__ y, const float* __restrict__ weights, int top,
                                   const float* __restrict__ shared, const float* __restrict__ logits, int ld_logits,
                                   int gate_col, float* __restrict__ resid, int width, const int* __restrict__ pair_pos) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  float g = 0.f;
  if (shared) g = 1.f / (1.f + expf(-logits[(size_t)t * ld_logits + gate_col]));
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float acc = 0.f;
    for (int x = 0; x < top; ++x) {
      const size_t pair = (size_t)t * top + x;
      acc = fmaf(weights[pair], y[(pair_pos ? (size_t)pair_pos[pair] : pair) * width + c], acc);
    }
    if (shared) acc = fmaf(g, shared[(size_t)t * width + c], acc);
    resid[(size_t)t * width + c] += acc;
  }
}

template <typename T>
__global__ void gelu_kernel(const T* __restrict__ x, T* __restrict__ y, long long n) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    y[i] = from_f32<T>(gelu_erf(to_f32(x[i])));
}

}  // namespace tllm

using namespace tllm;

extern "C" int tllm_moe_route(const float* logits, int ld, int n_experts, const float* correction, float scale, int top,
                              int* ids, float* weights, int n_tokens, int softmax, void* stream) {
  TLLM_REQUIRE(n_tokens > 0 && n_experts > 0 && top > 0 && top <= n_experts, "moe_route: %d of %d experts for %d tokens", top, n_experts, n_tokens);
  TLLM_REQUIRE(n_experts <= 32 * ROUTE_PER_LANE, "moe_route: %d experts (at most %d)", n_experts, 32 * ROUTE_PER_LANE);
  const int warps = 4;
  TLLM_LAUNCH("moe_route", moe_route_kernel, (unsigned)((n_tokens + warps - 1) / warps), warps * 32, 0, (cudaStream_t)stream,
              logits, ld, n_experts, correction, scale, top, ids, weights, n_tokens, softmax);
  return TLLM_OK;
}

extern "C" int tllm_moe_align(const int* ids, int n_pairs, int n_experts, int tile, int max_tiles, int* sorted_rows,
                              int* tile_expert, int* pair_pos, void* stream) {
  TLLM_REQUIRE(n_pairs > 0 && n_experts > 0 && tile > 0 && max_tiles > 0, "moe_align: empty input");
  TLLM_REQUIRE(n_experts <= 4096, "moe_align: %d experts (at most 4096)", n_experts);
  TLLM_LAUNCH("moe_align", moe_align_kernel, 1, 1024, (size_t)2 * n_experts * sizeof(int), (cudaStream_t)stream, ids, n_pairs,
              n_experts, tile, max_tiles, sorted_rows, tile_expert, pair_pos);
  return TLLM_OK;
}

// in: bfloat16 [rows, k] rows of ld_in values; out: bfloat16 [max_tiles * tile, k], contiguous.
extern "C" int tllm_moe_gather(const void* in, int ld_in, const int* sorted_rows, const int* tile_expert, int tile,
                               int max_tiles, int rows_per_input, void* out, int k, void* stream) {
  TLLM_REQUIRE(k > 0 && k % 8 == 0 && ld_in % 8 == 0 && ((uintptr_t)in & 15) == 0 && ((uintptr_t)out & 15) == 0,
               "moe_gather: rows of %d values (stride %d) must be multiples of 8 on 16-byte boundaries", k, ld_in);
  TLLM_REQUIRE(tile > 0 && max_tiles > 0 && rows_per_input > 0, "moe_gather: empty input");
  TLLM_LAUNCH("moe_gather", moe_gather_kernel, (unsigned)(max_tiles * tile), 128, 0, (cudaStream_t)stream, (const __nv_bfloat16*)in, ld_in,
              sorted_rows, tile_expert, tile, rows_per_input, (__nv_bfloat16*)out, k);
  return TLLM_OK;
}

template <typename T, typename TO>
static int moe_linear_launch(const void* in, int ld_in, const void* w, const int* sorted_rows, const int* tile_expert,
                             void* out, int n, int k, int rows_per_input, int tile, int max_tiles, int gelu, cudaStream_t s) {
  const dim3 grid((unsigned)max_tiles, (unsigned)((n + 63) / 64));
#define TLLM_MOE_CASE(TM, G)                                                                                          \
  TLLM_LAUNCH("moe_linear", (moe_linear_kernel<T, TO, TM, G>), grid, 256, 0, s, (const T*)in, ld_in, (const T*)w,      \
              sorted_rows, tile_expert, (TO*)out, n, k, rows_per_input)
  if (tile == 16) { if (gelu) TLLM_MOE_CASE(16, true); else TLLM_MOE_CASE(16, false); }
  else { if (gelu) TLLM_MOE_CASE(64, true); else TLLM_MOE_CASE(64, false); }
#undef TLLM_MOE_CASE
  return TLLM_OK;
}

// in: [rows, k] rows of ld_in values; w: [experts, n, k]; out: [pairs, n] of out_dtype.  use_mma != 0: bfloat16 products
// whose K and row stride are multiples of 8 run on the tensor cores; everything else on the FFMA kernel.
extern "C" int tllm_moe_linear(const void* in, int ld_in, const void* w, const int* sorted_rows, const int* tile_expert,
                               void* out, int n, int k, int rows_per_input, int tile, int max_tiles, int gelu, int dtype,
                               int out_dtype, int use_mma, void* stream) {
  TLLM_REQUIRE(n > 0 && k > 0 && rows_per_input > 0 && max_tiles > 0 && (tile == 16 || tile == 64 || tile == 128), "moe_linear: sizes do not fit (tile %d)", tile);
  TLLM_REQUIRE(tile != 128 || (dtype == TLLM_BF16 && use_mma && k % 8 == 0 && ld_in % 8 == 0 && ((uintptr_t)in & 15) == 0 && ((uintptr_t)w & 15) == 0),
               "moe_linear: tiles of 128 rows are the tensor-core kernel's");
  TLLM_REQUIRE(max_tiles <= 2147483647 && (n + 63) / 64 <= 65535, "moe_linear: the grid is too large");
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TLLM_BF16 && use_mma && k % 8 == 0 && ld_in % 8 == 0 && ((uintptr_t)in & 15) == 0 && ((uintptr_t)w & 15) == 0) {
    const dim3 grid((unsigned)max_tiles, (unsigned)((n + 127) / 128));
    TLLM_REQUIRE((n + 127) / 128 <= 65535, "moe_linear: the grid is too large");
#define TLLM_MOE_MMA(TO, BM, G)                                                                                           \
  do {                                                                                                                    \
    const size_t smem = sizeof(__nv_bfloat16) * (BM == 16 ? 4 : 3) * (BM + 128) * 40 + BM * sizeof(int);                   \
    static bool configured = false;                                                                                       \
    if (!configured) {                                                                                                    \
      cudaError_t e_ = cudaFuncSetAttribute(moe_linear_mma_kernel<TO, BM, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e_ != cudaSuccess) TLLM_FAIL(TLLM_ERR_CUDA, "moe_linear: %s", cudaGetErrorString(e_));                           \
      configured = true;                                                                                                  \
    }                                                                                                                     \
    TLLM_LAUNCH("moe_linear", (moe_linear_mma_kernel<TO, BM, G>), grid, 256, smem, s, (const __nv_bfloat16*)in, ld_in,     \
                (const __nv_bfloat16*)w, sorted_rows, tile_expert, (TO*)out, n, k, rows_per_input);                        \
  } while (0)
#define TLLM_MOE_MMA_TILES(TO)                                                                      \
  do {                                                                                              \
    if (tile == 16) { if (gelu) TLLM_MOE_MMA(TO, 16, true); else TLLM_MOE_MMA(TO, 16, false); }      \
    else if (tile == 64) { if (gelu) TLLM_MOE_MMA(TO, 64, true); else TLLM_MOE_MMA(TO, 64, false); } \
    else { if (gelu) TLLM_MOE_MMA(TO, 128, true); else TLLM_MOE_MMA(TO, 128, false); }               \
    return TLLM_OK;                                                                                 \
  } while (0)
    if (out_dtype == TLLM_BF16) TLLM_MOE_MMA_TILES(__nv_bfloat16);
    if (out_dtype == TLLM_F32) TLLM_MOE_MMA_TILES(float);
#undef TLLM_MOE_MMA_TILES
#undef TLLM_MOE_MMA
  }
  if (dtype == TLLM_F32 && out_dtype == TLLM_F32)
    return moe_linear_launch<float, float>(in, ld_in, w, sorted_rows, tile_expert, out, n, k, rows_per_input, tile, max_tiles, gelu, s);
  if (dtype == TLLM_BF16 && out_dtype == TLLM_BF16)
    return moe_linear_launch<__nv_bfloat16, __nv_bfloat16>(in, ld_in, w, sorted_rows, tile_expert, out, n, k, rows_per_input, tile, max_tiles, gelu, s);
  if (dtype == TLLM_BF16 && out_dtype == TLLM_F32)
    return moe_linear_launch<__nv_bfloat16, float>(in, ld_in, w, sorted_rows, tile_expert, out, n, k, rows_per_input, tile, max_tiles, gelu, s);
  TLLM_FAIL(TLLM_ERR_ARG, "moe_linear: dtype codes %d -> %d", dtype, out_dtype);
}

extern "C" int tllm_moe_combine(const float* y, const float* weights, int top, const float* shared, const float* logits,
                                int ld_logits, int gate_col, float* resid, int n_tokens, int width, const int* pair_pos,
                                void* stream) {
  TLLM_REQUIRE(n_tokens > 0 && width > 0 && top > 0, "moe_combine: empty input");
  TLLM_REQUIRE(!shared || logits, "moe_combine: a shared expert needs its gate's logits");
  TLLM_LAUNCH("moe_combine", moe_combine_kernel, (unsigned)n_tokens, width >= 1024 ? 256 : 128, 0, (cudaStream_t)stream, y, weights, top,
              shared, logits, ld_logits, gate_col, resid, width, pair_pos);
  return TLLM_OK;
}

extern "C" int tllm_gelu(const void* x, void* y, long long n, int dtype, void* stream) {
  TLLM_REQUIRE(n > 0, "gelu: empty input");
  const long long blocks = (n + 255) / 256;
  const unsigned grid = (unsigned)(blocks > 148 * 16 ? 148 * 16 : blocks);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TLLM_F32)
    TLLM_LAUNCH("gelu", gelu_kernel<float>, grid, 256, 0, s, (const float*)x, (float*)y, n);
  else if (dtype == TLLM_BF16)
    TLLM_LAUNCH("gelu", gelu_kernel<__nv_bfloat16>, grid, 256, 0, s, (const __nv_bfloat16*)x, (__nv_bfloat16*)y, n);
  else
    TLLM_FAIL(TLLM_ERR_ARG, "gelu: unknown dtype code %d", dtype);
  return TLLM_OK;
}
