// One small product per head in one launch:
//   out[t, h * o_hs + n] = sum_k a[t, h * a_hs + k] * w[h, n, k]        t < T, h < heads, n < N, k < K
// `a` and `out` are rows of tokens whose heads lie side by side (any row stride, any distance between heads), `w` is
// [heads, N, K] with rows contiguous.  It serves projections that differ from head to head and are too small to be
// worth a launch each: a latent attention's queries into the latent's space and its values out of it.
//
// head_linear_mma (bfloat16, K even, rows and heads of `a` at even offsets): a CTA of four warps owns 64 tokens x 64
//   outputs of one head; a warp 16 tokens x 64 outputs as eight m16n8k16 tiles.  The fragments are read straight from
//   global memory: a thread's two neighbouring values of A or W are one 32-bit load (W's K runs contiguously, which is
//   the column-major B the instruction takes), a head's weights stay in L1.  Steps of at most 32 tokens give a CTA 16
//   tokens and each of its warps 16 of the 64 outputs instead.  Sums are 32-bit, an output's sum runs over ascending
//   k in steps of 16 whatever its tile, so its bits do not depend on the batch.
// head_linear_simt (both dtypes, every size): tiles of 16 tokens x 64 outputs x 32 k through shared memory, four
//   tokens of one output per thread, every output one chain of fmaf over ascending k.
#include <cstdint>

#include "common.cuh"

TLLM_DEFINE_LAST_ERROR

namespace tllm {

struct HeadLinearArgs {
  const void* a;
  long long a_ld;      // values between token rows of a
  int a_hs;            // values between heads inside a row
  const void* w;       // [heads, n, k]
  void* out;
  long long o_ld;
  int o_hs;
  int tokens, heads, n, k;
};

__device__ __forceinline__ void mma_bf16_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// FEW = false: the CTA's four warps take 16 token rows each and all 64 outputs.  FEW = true (steps of few tokens): the
// CTA has 16 token rows and its warps 16 outputs each, so that a decode step's weights are fetched by four warps.
template <typename TO, bool FEW>
__global__ void __launch_bounds__(128) head_linear_mma_kernel(HeadLinearArgs p) {
  constexpr int NT = FEW ? 2 : 8;     // tiles of 8 outputs per warp
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tg = lane & 3;
  const int h = blockIdx.z;
  const int row0 = FEW ? blockIdx.y * 16 : blockIdx.y * 64 + warp * 16;
  const int n0 = blockIdx.x * 64 + (FEW ? warp * 16 : 0);
  if (row0 >= p.tokens || n0 >= p.n) return;
  const __nv_bfloat16* a = (const __nv_bfloat16*)p.a + (size_t)h * p.a_hs;
  const __nv_bfloat16* w = (const __nv_bfloat16*)p.w + (size_t)h * p.n * p.k;
  const int r_lo = row0 + g, r_hi = row0 + g + 8;
  const bool lo_ok = r_lo < p.tokens, hi_ok = r_hi < p.tokens;
  const __nv_bfloat16* a_lo = a + (size_t)r_lo * p.a_ld;
  const __nv_bfloat16* a_hi = a + (size_t)r_hi * p.a_ld;
  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;
#pragma unroll 4
  for (int k0 = 0; k0 < p.k; k0 += 16) {
    const int ka = k0 + 2 * tg, kb = ka + 8;     // K is even: a pair is inside or outside as a whole
    uint32_t fa[4];
    fa[0] = (lo_ok && ka < p.k) ? *(const uint32_t*)(a_lo + ka) : 0u;
    fa[1] = (hi_ok && ka < p.k) ? *(const uint32_t*)(a_hi + ka) : 0u;
    fa[2] = (lo_ok && kb < p.k) ? *(const uint32_t*)(a_lo + kb) : 0u;
    fa[3] = (hi_ok && kb < p.k) ? *(const uint32_t*)(a_hi + kb) : 0u;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      const int n = n0 + j * 8 + g;
      const __nv_bfloat16* wr = w + (size_t)n * p.k;
      const uint32_t b0 = (n < p.n && ka < p.k) ? *(const uint32_t*)(wr + ka) : 0u;
      const uint32_t b1 = (n < p.n && kb < p.k) ? *(const uint32_t*)(wr + kb) : 0u;
      mma_bf16_16816(acc[j], fa, b0, b1);
    }
  }
  TO* out = (TO*)p.out + (size_t)h * p.o_hs;
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const int n = n0 + j * 8 + 2 * tg;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      if (n + i >= p.n) continue;
      if (lo_ok) out[(size_t)r_lo * p.o_ld + n + i] = from_f32<TO>(acc[j][i]);
      if (hi_ok) out[(size_t)r_hi * p.o_ld + n + i] = from_f32<TO>(acc[j][2 + i]);
    }
  }
}

template <typename T, typename TO>
__global__ void __launch_bounds__(256) head_linear_simt_kernel(HeadLinearArgs p) {
  __shared__ float as[16][33], wsh[32][65];
  pdl_trigger();
  pdl_wait();
  const int tid = threadIdx.x;
  const int h = blockIdx.z;
  const int row0 = blockIdx.y * 16, n0 = blockIdx.x * 64;
  const T* a = (const T*)p.a + (size_t)h * p.a_hs;
  const T* w = (const T*)p.w + (size_t)h * p.n * p.k;
  const int nl = tid & 63, tq = tid >> 6;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k0 = 0; k0 < p.k; k0 += 32) {
    for (int i = tid; i < 16 * 32; i += 256) {
      const int r = i >> 5, kk = i & 31;
      as[r][kk] = (row0 + r < p.tokens && k0 + kk < p.k) ? to_f32(a[(size_t)(row0 + r) * p.a_ld + k0 + kk]) : 0.f;
    }
    for (int i = tid; i < 64 * 32; i += 256) {
      const int n = i >> 5, kk = i & 31;
      wsh[kk][n] = (n0 + n < p.n && k0 + kk < p.k) ? to_f32(w[(size_t)(n0 + n) * p.k + k0 + kk]) : 0.f;
    }
    __syncthreads();
    const int kn = min(32, p.k - k0);    // zeros past K would not change a sum, but the chain stays K long
    for (int kk = 0; kk < kn; ++kk) {
      const float wv = wsh[kk][nl];
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[j] = fmaf(as[tq * 4 + j][kk], wv, acc[j]);
    }
    __syncthreads();
  }
  if (n0 + nl >= p.n) return;
  TO* out = (TO*)p.out + (size_t)h * p.o_hs;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int r = row0 + tq * 4 + j;
    if (r < p.tokens) out[(size_t)r * p.o_ld + n0 + nl] = from_f32<TO>(acc[j]);
  }
}

}  // namespace tllm

using namespace tllm;

// dtype: of a and w; out_dtype: of out (the same, or float32).  tensor_cores != 0 lets bfloat16 inputs whose sizes
// allow it take the mma.sync kernel.
extern "C" int tllm_head_linear(const void* a, long long a_ld, int a_hs, const void* w, void* out, long long o_ld, int o_hs,
                                int tokens, int heads, int n, int k, int dtype, int out_dtype, int tensor_cores,
                                void* stream) {
  TLLM_REQUIRE(tokens > 0 && heads > 0 && heads <= 65535 && n > 0 && k > 0 && a && w && out,
               "head_linear: %d tokens, %d heads, %d outputs of %d inputs", tokens, heads, n, k);
  TLLM_REQUIRE((dtype == TLLM_F32 || dtype == TLLM_BF16) && (out_dtype == dtype || out_dtype == TLLM_F32),
               "head_linear: dtype codes %d -> %d", dtype, out_dtype);
  HeadLinearArgs p;
  p.a = a; p.a_ld = a_ld; p.a_hs = a_hs; p.w = w; p.out = out; p.o_ld = o_ld; p.o_hs = o_hs;
  p.tokens = tokens; p.heads = heads; p.n = n; p.k = k;
  cudaStream_t s = (cudaStream_t)stream;
  const bool mma = tensor_cores && dtype == TLLM_BF16 && k % 2 == 0 && a_ld % 2 == 0 && a_hs % 2 == 0 &&
                   ((uintptr_t)a % 4) == 0 && ((uintptr_t)w % 4) == 0;
  if (mma) {
    const bool few = tokens <= 32;
    const long long gy = few ? ((long long)tokens + 15) / 16 : ((long long)tokens + 63) / 64;
    TLLM_REQUIRE(gy <= 65535, "head_linear: %d tokens exceed the grid", tokens);
    const dim3 grid((n + 63) / 64, (unsigned)gy, heads);
    if (few && out_dtype == TLLM_F32) TLLM_LAUNCH("head_linear_mma", (head_linear_mma_kernel<float, true>), grid, 128, 0, s, p);
    else if (few) TLLM_LAUNCH("head_linear_mma", (head_linear_mma_kernel<__nv_bfloat16, true>), grid, 128, 0, s, p);
    else if (out_dtype == TLLM_F32) TLLM_LAUNCH("head_linear_mma", (head_linear_mma_kernel<float, false>), grid, 128, 0, s, p);
    else TLLM_LAUNCH("head_linear_mma", (head_linear_mma_kernel<__nv_bfloat16, false>), grid, 128, 0, s, p);
    return TLLM_OK;
  }
  const long long gy = ((long long)tokens + 15) / 16;
  TLLM_REQUIRE(gy <= 65535, "head_linear: %d tokens exceed the grid", tokens);
  const dim3 grid((n + 63) / 64, (unsigned)gy, heads);
  if (dtype == TLLM_F32) TLLM_LAUNCH("head_linear_simt", (head_linear_simt_kernel<float, float>), grid, 256, 0, s, p);
  else if (out_dtype == TLLM_F32) TLLM_LAUNCH("head_linear_simt", (head_linear_simt_kernel<__nv_bfloat16, float>), grid, 256, 0, s, p);
  else TLLM_LAUNCH("head_linear_simt", (head_linear_simt_kernel<__nv_bfloat16, __nv_bfloat16>), grid, 256, 0, s, p);
  return TLLM_OK;
}
