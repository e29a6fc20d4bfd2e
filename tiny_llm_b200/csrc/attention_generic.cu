// Attention of the step's queries over the paged cache on the CUDA cores, any key size and any value
// size up to 256 (the two may differ; key rows whose bytes are a multiple of 16 are read with 16-byte loads), any number of heads and groups, any
// page size.  It is the attention of the true 32-bit path and the fallback of the bfloat16 path.
//
// Heads.  A query head has `maps` score maps, each an attention of its own over the same values: the
// query rows of a token are laid out [head][map][kd], the key rows [key/value head][map][kd], the
// value rows [key/value head][vd]; map m of query head h reads key row (h / group) * maps + m and
// value row h / group, and the output rows are [head][map][vd].  maps = 1 is ordinary grouped-query
// attention.  The output is of the cache's type or float32 (for a caller that combines the maps).
//
// The keys a query at position p sees are j in [lo, p] with lo = max(0, p - window + 1) when there is a
// window and lo >= (p / chunk) * chunk when keys are visible inside a chunk of positions only (chunks
// are counted from position 0 of the sequence).  They are walked in
// tiles of 32 that start at multiples of 32 of the absolute position.  Tile number i (= j / 32) belongs
// to lane i mod 8 of eight running softmaxes (m, l, o) in 32-bit, each of which takes its tiles in
// ascending order; at the end the eight are merged in the order 0..7.  So the order of every sum is a
// function of p alone: the result does not depend on how the request's tokens were cut into steps, on
// the rest of the batch or on the page ids.  Two launches of the same arithmetic: with many (token,
// head) pairs one warp carries all eight softmaxes of a pair (prompts); with few, eight warps carry
// one each and merge through shared memory (decoded tokens over a long context, where one warp per
// pair would leave most of the GPU idle and walk thousands of keys as one chain of memory latencies).
// Every step of both is written with explicit fmaf / __fmul_rn, so that the two compile to the same
// operations and give the same bits.
// Reference counterpart: tiny_llm/ops/cuda/flash_attention.cu:338-442 (64-key tiles,
// one lane per key, P.V by shuffles), whose mask compares a chunk-local query index with the
// absolute key index (:63-66, :402-405).
#include <math_constants.h>

#include "common.cuh"

TLLM_DEFINE_LAST_ERROR

namespace tllm {

constexpr int WARPS = 4;
constexpr int MAX_HD = 256;

// Where the rows of the cache lie and which keys are visible; `nq` and `nk` count (head, map) rows.
struct Geometry {
  int nq, nk, maps, kd, vd, page_size, window, chunk;
  int kvec;   // key rows are read with 16-byte loads (their size and strides allow it); else value by value, same order
  long long k_page_stride, k_head_stride, v_page_stride, v_head_stride;
};
__device__ __forceinline__ int lowest_key(const Geometry& g, int p) {
  int lo = g.window > 0 ? max(0, p - g.window + 1) : 0;
  if (g.chunk > 0) lo = max(lo, (p / g.chunk) * g.chunk);
  return lo;
}

template <typename T> struct Vec;            // 16-byte vectors of the cache rows
template <> struct Vec<float> { static constexpr int N = 4; };
template <> struct Vec<__nv_bfloat16> { static constexpr int N = 8; };

__device__ __forceinline__ void load16(const float* p, float* dst) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
}
__device__ __forceinline__ void load16(const __nv_bfloat16* p, float* dst) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    dst[2 * i] = f.x; dst[2 * i + 1] = f.y;
  }
}

constexpr int WAYS = 8;   // running softmaxes per (token, head); a constant of the arithmetic, not a tuning knob

template <int OD>   // OD * 32 >= head size: the output values of a lane
struct Softmax {
  float m, l;
  float o[OD];
};

// One tile of 32 keys starting at j0 into the running softmax `st` (all lanes of the warp).
template <typename T, int OD>
__device__ __forceinline__ void attend_tile(Softmax<OD>& st, int j0, int lo, int p, const float* q_row, const T* kcache,
                                            const T* vcache, const int* table, int max_blocks, int kh, int vh,
                                            const Geometry& g, int lane) {
  const int hd = g.kd, vd = g.vd, page_size = g.page_size;
  const int j = j0 + lane;
  bool valid = j >= lo && j <= p && j / page_size < max_blocks;
  const int page = valid ? table[j / page_size] : -1;
  valid = valid && page >= 0;   // a table entry that names no page is never followed
  long long row_off = 0;
  float s = -CUDART_INF_F;
  if (valid) {
    row_off = (long long)page * g.v_page_stride + (long long)vh * g.v_head_stride + (long long)(j % page_size) * vd;
    const T* krow = kcache + (long long)page * g.k_page_stride + (long long)kh * g.k_head_stride + (long long)(j % page_size) * hd;
    float acc = 0.f;
    if (g.kvec) {
#pragma unroll 4
      for (int d = 0; d < hd; d += Vec<T>::N) {
        float kv[Vec<T>::N];
        load16(krow + d, kv);
#pragma unroll
        for (int e = 0; e < Vec<T>::N; ++e) acc = fmaf(q_row[d + e], kv[e], acc);
      }
    } else {
      for (int d = 0; d < hd; ++d) acc = fmaf(q_row[d], to_f32(krow[d]), acc);
    }
    s = acc;
  }
  const float m_new = fmaxf(st.m, warp_max(s));
  const float m_ref = m_new == -CUDART_INF_F ? 0.f : m_new;   // a tile without a visible key changes nothing
  const float pr = valid ? expf(s - m_ref) : 0.f;
  const float corr = expf(st.m - m_ref);           // 0 on the first tile (m = -inf)
  st.l = fmaf(st.l, corr, warp_sum(pr));
  st.m = m_new;
#pragma unroll
  for (int i = 0; i < OD; ++i) st.o[i] = __fmul_rn(st.o[i], corr);
  const int last = min(31, p - j0);
  const int first = max(0, lo - j0);
  for (int kk = first; kk <= last; ++kk) {
    const float pk = __shfl_sync(0xffffffffu, pr, kk);
    if (pk == 0.f) continue;   // uniform across the warp: nothing to add, and the row may name no page
    const long long off = __shfl_sync(0xffffffffu, row_off, kk);
    const T* vrow = vcache + off;
#pragma unroll
    for (int i = 0; i < OD; ++i) {
      const int d = lane + 32 * i;
      if (d < vd) st.o[i] = fmaf(pk, to_f32(vrow[d]), st.o[i]);
    }
  }
}

// The merge of the eight softmaxes, way 0 first: `m`, `l`, `o` of way w are read through the three functions.
template <int OD, typename FM, typename FL, typename FO>
__device__ __forceinline__ void merge_ways(FM way_m, FL way_l, FO way_o, float* o_out, float& l_out, float& m_out) {
  float mx = -CUDART_INF_F;
#pragma unroll
  for (int w = 0; w < WAYS; ++w) mx = fmaxf(mx, way_m(w));
  const float m_ref = mx == -CUDART_INF_F ? 0.f : mx;
  m_out = m_ref;
  l_out = 0.f;
#pragma unroll
  for (int i = 0; i < OD; ++i) o_out[i] = 0.f;
#pragma unroll
  for (int w = 0; w < WAYS; ++w) {
    const float f = expf(way_m(w) - m_ref);   // 0 for a way that saw no key
    l_out = fmaf(way_l(w), f, l_out);
#pragma unroll
    for (int i = 0; i < OD; ++i) o_out[i] = fmaf(way_o(w, i), f, o_out[i]);
  }
}

// What the merged sums are multiplied by: 1 / l, or, with a sink (a learned score per head that joins the softmax's
// denominator and has no value), 1 / (l + exp(sink - m)) with both terms taken against the larger of m and the sink.
__device__ __forceinline__ float inverse_sum(float l, float m, const float* sink, int head) {
  if (sink == nullptr) return 1.f / l;
  const float sk = sink[head];
  const float top = fmaxf(m, sk);
  const float f = expf(m - top);
  return f / fmaf(l, f, expf(sk - top));
}

// The same tile for up to GH query heads that share the key/value head: every key row and value row is fetched once
// for all of them.  Head by head the operations are those of attend_tile, in the same order.
constexpr int GH = 4;

template <typename T, int OD>
__device__ __forceinline__ void attend_tile_grouped(Softmax<OD> (&st)[GH], int nh, int j0, int lo, int p,
                                                    const float (*q_rows)[OD * 32], const T* kcache, const T* vcache,
                                                    const int* table, int max_blocks, int kh, int vh,
                                                    const Geometry& g, int lane) {
  const int hd = g.kd, vd = g.vd, page_size = g.page_size;
  const int j = j0 + lane;
  bool valid = j >= lo && j <= p && j / page_size < max_blocks;
  const int page = valid ? table[j / page_size] : -1;
  valid = valid && page >= 0;
  long long row_off = 0;
  float s[GH];
#pragma unroll
  for (int i = 0; i < GH; ++i) s[i] = -CUDART_INF_F;
  if (valid) {
    row_off = (long long)page * g.v_page_stride + (long long)vh * g.v_head_stride + (long long)(j % page_size) * vd;
    const T* krow = kcache + (long long)page * g.k_page_stride + (long long)kh * g.k_head_stride + (long long)(j % page_size) * hd;
    float acc[GH];
#pragma unroll
    for (int i = 0; i < GH; ++i) acc[i] = 0.f;
    if (g.kvec) {
#pragma unroll 2
      for (int d = 0; d < hd; d += Vec<T>::N) {
        float kv[Vec<T>::N];
        load16(krow + d, kv);
#pragma unroll
        for (int i = 0; i < GH; ++i)
#pragma unroll
          for (int e = 0; e < Vec<T>::N; ++e) acc[i] = fmaf(q_rows[i][d + e], kv[e], acc[i]);
      }
    } else {
      for (int d = 0; d < hd; ++d) {
        const float kvd = to_f32(krow[d]);
#pragma unroll
        for (int i = 0; i < GH; ++i) acc[i] = fmaf(q_rows[i][d], kvd, acc[i]);
      }
    }
#pragma unroll
    for (int i = 0; i < GH; ++i) s[i] = acc[i];
  }
  float pr[GH];
#pragma unroll
  for (int i = 0; i < GH; ++i) {
    pr[i] = 0.f;
    if (i < nh) {
      const float m_new = fmaxf(st[i].m, warp_max(s[i]));
      const float m_ref = m_new == -CUDART_INF_F ? 0.f : m_new;
      pr[i] = valid ? expf(s[i] - m_ref) : 0.f;
      const float corr = expf(st[i].m - m_ref);
      st[i].l = fmaf(st[i].l, corr, warp_sum(pr[i]));
      st[i].m = m_new;
#pragma unroll
      for (int x = 0; x < OD; ++x) st[i].o[x] = __fmul_rn(st[i].o[x], corr);
    }
  }
  const int last = min(31, p - j0);
  const int first = max(0, lo - j0);
  for (int kk = first; kk <= last; ++kk) {
    float pk[GH];
    bool any = false;
#pragma unroll
    for (int i = 0; i < GH; ++i) {
      pk[i] = __shfl_sync(0xffffffffu, pr[i], kk);
      any = any || pk[i] != 0.f;
    }
    if (!any) continue;   // uniform across the warp: nothing to add, and the row may name no page
    const long long off = __shfl_sync(0xffffffffu, row_off, kk);
    const T* vrow = vcache + off;
#pragma unroll
    for (int x = 0; x < OD; ++x) {
      const int d = lane + 32 * x;
      if (d < vd) {
        const float v = to_f32(vrow[d]);
#pragma unroll
        for (int i = 0; i < GH; ++i)
          if (pk[i] != 0.f) st[i].o[x] = fmaf(pk[i], v, st[i].o[x]);
      }
    }
  }
}

// Many (token, head) pairs (prompts): one warp per (token, key row, up to GH of the query rows that read it).  The eight
// softmaxes are walked one after the other (way w over its own tiles in ascending order, as everywhere), their results
// parked in shared memory and merged per head in the order 0..7: the arithmetic of every head is that of the other two
// launches, and the keys and values of a tile are fetched once for the heads of the group instead of once per head
// (with one warp per pair the kernel was bound by those fetches: 34 GB through L2 per layer of a 2,048-token prompt).
template <int OD> struct GroupedWarps { static constexpr int N = OD <= 2 ? 4 : (OD <= 4 ? 2 : 1); };

template <typename T, typename TO, int OD>
__global__ void __launch_bounds__(GroupedWarps<OD>::N * 32)
paged_attention_grouped_kernel(const T* __restrict__ q, int q_row_stride, const T* __restrict__ kcache,
                               const T* __restrict__ vcache, const int* __restrict__ block_table,
                               int max_blocks, const int* __restrict__ token_request,
                               const int* __restrict__ positions, TO* __restrict__ out, int n_tokens,
                               Geometry g, float scale, const float* __restrict__ sink) {
  constexpr int GW = GroupedWarps<OD>::N;
  __shared__ __align__(16) float q_s[GW][GH][OD * 32];
  __shared__ float way_s[GW][WAYS][GH][OD * 32 + 2];
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = g.nq, nk = g.nk, hd = g.kd, vd = g.vd, maps = g.maps;
  const int group = nq / nk, chunks = (group + GH - 1) / GH;
  const long long task = (long long)blockIdx.x * GW + warp;
  if (task >= (long long)n_tokens * nk * chunks) return;
  const int t = (int)(task / (nk * chunks)), rem = (int)(task % (nk * chunks));
  const int kh = rem / chunks, h0 = (rem % chunks) * GH, nh = min(GH, group - h0);
  const int kvh = kh / maps, map = kh % maps;   // query row of head h, map m: (h * maps + m)
  const int vh = kvh;
  const int req = token_request[t];
  const int p = positions[t];
  const int lo = lowest_key(g, p);
  const int* table = block_table + (size_t)req * max_blocks;
  for (int i = 0; i < nh; ++i) {
    const T* qrow = q + (size_t)t * q_row_stride + (size_t)((kvh * group + h0 + i) * maps + map) * hd;
    for (int d = lane; d < hd; d += 32) q_s[warp][i][d] = to_f32(qrow[d]) * scale;
  }
  for (int i = nh; i < GH; ++i)
    for (int d = lane; d < hd; d += 32) q_s[warp][i][d] = 0.f;
  __syncwarp();

  const int first_group = (lo / (32 * WAYS)) * (32 * WAYS);
  for (int w = 0; w < WAYS; ++w) {
    Softmax<OD> st[GH];
#pragma unroll
    for (int i = 0; i < GH; ++i) {
      st[i].m = -CUDART_INF_F; st[i].l = 0.f;
#pragma unroll
      for (int x = 0; x < OD; ++x) st[i].o[x] = 0.f;
    }
    for (int j0 = first_group + w * 32; j0 <= p; j0 += 32 * WAYS)
      if (j0 + 31 >= lo)
        attend_tile_grouped<T, OD>(st, nh, j0, lo, p, q_s[warp], kcache, vcache, table, max_blocks, kh, vh, g, lane);
#pragma unroll
    for (int i = 0; i < GH; ++i) {
      if (lane == 0) { way_s[warp][w][i][OD * 32] = st[i].m; way_s[warp][w][i][OD * 32 + 1] = st[i].l; }
#pragma unroll
      for (int x = 0; x < OD; ++x) way_s[warp][w][i][lane + 32 * x] = st[i].o[x];
    }
  }
  __syncwarp();
  for (int i = 0; i < nh; ++i) {
    float o[OD], l, mx;
    merge_ways<OD>([&](int w) { return way_s[warp][w][i][OD * 32]; }, [&](int w) { return way_s[warp][w][i][OD * 32 + 1]; },
                   [&](int w, int x) { return way_s[warp][w][i][lane + 32 * x]; }, o, l, mx);
    TO* orow = out + (size_t)t * nq * vd + (size_t)((kvh * group + h0 + i) * maps + map) * vd;
    const float inv = inverse_sum(l, mx, sink, kvh * group + h0 + i);
#pragma unroll
    for (int x = 0; x < OD; ++x) {
      const int d = lane + 32 * x;
      if (d < vd) orow[d] = from_f32<TO>(o[x] * inv);
    }
  }
}

// SPLIT = false: WARPS (token, head) pairs per CTA, one warp each, eight softmaxes in its registers.
// SPLIT = true: one pair per CTA of eight warps, warp w carries softmax w.
template <typename T, typename TO, bool SPLIT, int OD>
__global__ void __launch_bounds__(SPLIT ? WAYS * 32 : WARPS * 32)
paged_attention_generic_kernel(const T* __restrict__ q, int q_row_stride, const T* __restrict__ kcache,
                               const T* __restrict__ vcache, const int* __restrict__ block_table,
                               int max_blocks, const int* __restrict__ token_request,
                               const int* __restrict__ positions, TO* __restrict__ out, int n_tokens,
                               Geometry g, float scale, const float* __restrict__ sink) {
  __shared__ __align__(16) float q_s[SPLIT ? 1 : WARPS][MAX_HD];
  __shared__ float merge_s[SPLIT ? WAYS : 1][SPLIT ? OD * 32 + 2 : 1];
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = g.nq, nk = g.nk, hd = g.kd, vd = g.vd, maps = g.maps;
  const long long task = SPLIT ? (long long)blockIdx.x : (long long)blockIdx.x * WARPS + warp;
  if (task >= (long long)n_tokens * nq) return;
  const int t = (int)(task / nq), h = (int)(task % nq);   // h: the (head, map) row of the queries
  const int vh = (h / maps) / (nq / nk);
  const int kh = vh * maps + h % maps;
  const int req = token_request[t];
  const int p = positions[t];
  const int lo = lowest_key(g, p);
  const int* table = block_table + (size_t)req * max_blocks;

  const T* qrow = q + (size_t)t * q_row_stride + (size_t)h * hd;
  float* q_row = q_s[SPLIT ? 0 : warp];
  if (SPLIT) {
    for (int d = threadIdx.x; d < hd; d += WAYS * 32) q_row[d] = to_f32(qrow[d]) * scale;
    __syncthreads();
  } else {
    for (int d = lane; d < hd; d += 32) q_row[d] = to_f32(qrow[d]) * scale;
    __syncwarp();
  }

  const int first_group = (lo / (32 * WAYS)) * (32 * WAYS);   // tile numbers are absolute: way = (j0 / 32) % WAYS
  float o[OD], l, mx;
  if (SPLIT) {
    Softmax<OD> st;
    st.m = -CUDART_INF_F; st.l = 0.f;
#pragma unroll
    for (int i = 0; i < OD; ++i) st.o[i] = 0.f;
    for (int j0 = first_group + warp * 32; j0 <= p; j0 += 32 * WAYS)
      if (j0 + 31 >= lo)
        attend_tile(st, j0, lo, p, q_row, kcache, vcache, table, max_blocks, kh, vh, g, lane);
    if (lane == 0) { merge_s[warp][OD * 32] = st.m; merge_s[warp][OD * 32 + 1] = st.l; }
#pragma unroll
    for (int i = 0; i < OD; ++i)
      if (lane + 32 * i < vd) merge_s[warp][lane + 32 * i] = st.o[i];
    __syncthreads();
    if (warp != 0) return;
    merge_ways<OD>([&](int w) { return merge_s[w][OD * 32]; }, [&](int w) { return merge_s[w][OD * 32 + 1]; },
               [&](int w, int i) { return lane + 32 * i < vd ? merge_s[w][lane + 32 * i] : 0.f; }, o, l, mx);
  } else {
    Softmax<OD> st[WAYS];
#pragma unroll
    for (int w = 0; w < WAYS; ++w) {
      st[w].m = -CUDART_INF_F; st[w].l = 0.f;
#pragma unroll
      for (int i = 0; i < OD; ++i) st[w].o[i] = 0.f;
    }
    for (int g0 = first_group; g0 <= p; g0 += 32 * WAYS) {
#pragma unroll
      for (int w = 0; w < WAYS; ++w) {
        const int j0 = g0 + w * 32;
        if (j0 <= p && j0 + 31 >= lo)
          attend_tile(st[w], j0, lo, p, q_row, kcache, vcache, table, max_blocks, kh, vh, g, lane);
      }
    }
    merge_ways<OD>([&](int w) { return st[w].m; }, [&](int w) { return st[w].l; }, [&](int w, int i) { return st[w].o[i]; }, o, l, mx);
  }
  TO* orow = out + (size_t)t * nq * vd + (size_t)h * vd;
  const float inv = inverse_sum(l, mx, sink, h / maps);
#pragma unroll
  for (int i = 0; i < OD; ++i) {
    const int d = lane + 32 * i;
    if (d < vd) orow[d] = from_f32<TO>(o[i] * inv);
  }
}

template <typename T, typename TO>
static int launch_attention(const void* q, int q_row_stride, const void* kcache, const void* vcache, const int* block_table,
                            int max_blocks, const int* token_request, const int* positions, void* out, int n_tokens,
                            const Geometry& g, float scale, const float* sink, bool split, bool grouped, int od,
                            long long blocks, cudaStream_t s) {
#define TLLM_ATT_GENERIC(SPLIT_, OD_)                                                                                  \
  TLLM_LAUNCH("paged_attention_generic", (paged_attention_generic_kernel<T, TO, SPLIT_, OD_>), (unsigned)blocks,       \
              (SPLIT_ ? WAYS : WARPS) * 32, 0, s, (const T*)q, q_row_stride, (const T*)kcache, (const T*)vcache,       \
              block_table, max_blocks, token_request, positions, (TO*)out, n_tokens, g, scale, sink)
#define TLLM_ATT_GROUPED(OD_)                                                                                          \
  TLLM_LAUNCH("paged_attention_grouped", (paged_attention_grouped_kernel<T, TO, OD_>), (unsigned)blocks,               \
              GroupedWarps<OD_>::N * 32, 0, s, (const T*)q, q_row_stride, (const T*)kcache, (const T*)vcache,          \
              block_table, max_blocks, token_request, positions, (TO*)out, n_tokens, g, scale, sink)
  if (split) {
    if (od == 2) TLLM_ATT_GENERIC(true, 2); else if (od == 4) TLLM_ATT_GENERIC(true, 4); else TLLM_ATT_GENERIC(true, 8);
  } else if (grouped) {
    if (od == 2) TLLM_ATT_GROUPED(2); else if (od == 4) TLLM_ATT_GROUPED(4); else TLLM_ATT_GROUPED(8);
  } else {
    if (od == 2) TLLM_ATT_GENERIC(false, 2); else if (od == 4) TLLM_ATT_GENERIC(false, 4); else TLLM_ATT_GENERIC(false, 8);
  }
#undef TLLM_ATT_GROUPED
#undef TLLM_ATT_GENERIC
  return TLLM_OK;
}

}  // namespace tllm

using namespace tllm;

// Attention with `maps` score maps per head and key rows of `kd`, value rows of `vd` values.  `nq` query heads and
// `nkv` key/value heads; the key cache holds nkv * maps rows per slot, the value cache nkv.  `chunk` > 0: keys are
// visible inside the query's chunk of positions only.  out_f32 != 0: the output rows are float32 whatever the cache's type.
// `sink` (float32, one per query head, or null): exp(sink) joins every softmax's denominator of that head.
extern "C" int tllm_paged_attention_maps(const void* q, int q_row_stride, const void* kcache, const void* vcache,
                                         const int* block_table, int max_blocks, const int* token_request,
                                         const int* positions, void* out, int n_tokens, int nq, int nkv, int maps, int kd,
                                         int vd, int page_size, long long k_page_stride, long long k_head_stride,
                                         long long v_page_stride, long long v_head_stride, float scale, int window,
                                         int chunk, int dtype, int out_f32, int split_override, const float* sink,
                                         void* stream) {
  TLLM_REQUIRE(n_tokens > 0 && nq > 0 && nkv > 0 && nq % nkv == 0 && maps > 0,
               "attention: %d tokens, %d heads, %d key/value heads (heads must be a multiple of key/value heads)", n_tokens, nq, nkv);
  TLLM_REQUIRE(kd >= 1 && kd <= MAX_HD && vd >= 1 && vd <= MAX_HD,
               "attention: key size %d / value size %d is not built (both up to %d)", kd, vd, MAX_HD);
  TLLM_REQUIRE(page_size > 0 && max_blocks > 0 && window >= 0 && chunk >= 0, "attention: page size %d, %d blocks, window %d, chunk %d", page_size, max_blocks, window, chunk);
  const int elem = dtype == TLLM_F32 ? 4 : 2;
  TLLM_REQUIRE(dtype == TLLM_F32 || dtype == TLLM_BF16, "attention: unknown dtype code %d", dtype);
  Geometry g;
  g.kvec = (kd * elem) % 16 == 0 && ((size_t)kcache % 16) == 0 && (k_page_stride * elem) % 16 == 0 && (k_head_stride * elem) % 16 == 0;
  g.nq = nq * maps; g.nk = nkv * maps; g.maps = maps; g.kd = kd; g.vd = vd; g.page_size = page_size; g.window = window;
  g.chunk = chunk; g.k_page_stride = k_page_stride; g.k_head_stride = k_head_stride; g.v_page_stride = v_page_stride;
  g.v_head_stride = v_head_stride;
  const long long tasks = (long long)n_tokens * g.nq;
  // few pairs (decoded tokens): eight warps per pair; the result is the same to the bit
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    TLLM_FAIL(TLLM_ERR_CUDA, "attention: cannot read the number of SMs");
  // split_override: -1 by the number of pairs; 1 eight warps per pair; 0 one warp per (token, key row, four query rows);
  // 2 one warp per pair (the plainest form, kept for comparison: all give the same bits)
  const bool split = split_override >= 0 ? split_override == 1 : tasks <= 8LL * sms;
  const bool grouped = !split && split_override != 2;
  const int hd = kd > vd ? kd : vd;
  const int od = hd <= 64 ? 2 : (hd <= 128 ? 4 : 8);
  const int gw = od <= 2 ? 4 : (od <= 4 ? 2 : 1);
  const long long gtasks = (long long)n_tokens * g.nk * ((nq / nkv + GH - 1) / GH);
  const long long blocks = split ? tasks : (grouped ? (gtasks + gw - 1) / gw : (tasks + WARPS - 1) / WARPS);
  TLLM_REQUIRE(blocks <= 2147483647LL, "attention: %lld (token, head) pairs exceed the grid", tasks);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TLLM_F32)
    return launch_attention<float, float>(q, q_row_stride, kcache, vcache, block_table, max_blocks, token_request, positions, out,
                                          n_tokens, g, scale, sink, split, grouped, od, blocks, s);
  if (out_f32)
    return launch_attention<__nv_bfloat16, float>(q, q_row_stride, kcache, vcache, block_table, max_blocks, token_request,
                                                  positions, out, n_tokens, g, scale, sink, split, grouped, od, blocks, s);
  return launch_attention<__nv_bfloat16, __nv_bfloat16>(q, q_row_stride, kcache, vcache, block_table, max_blocks, token_request,
                                                        positions, out, n_tokens, g, scale, sink, split, grouped, od, blocks, s);
}

extern "C" int tllm_paged_attention_generic(const void* q, int q_row_stride, const void* kcache, const void* vcache,
                                            const int* block_table, int max_blocks, const int* token_request,
                                            const int* positions, void* out, int n_tokens, int nq, int nkv, int hd,
                                            int page_size, long long page_stride, long long head_stride,
                                            float scale, int window, int dtype, int split_override, void* stream) {
  TLLM_REQUIRE(hd >= 16 && hd <= MAX_HD && hd % 16 == 0,
               "attention: head size %d is not built (multiples of 16 up to %d are)", hd, MAX_HD);
  const int elem = dtype == TLLM_F32 ? 4 : 2;
  TLLM_REQUIRE(((size_t)vcache % 16) == 0 && (page_stride * elem) % 16 == 0 && (head_stride * elem) % 16 == 0,
               "attention: cache rows must be 16-byte aligned");
  return tllm_paged_attention_maps(q, q_row_stride, kcache, vcache, block_table, max_blocks, token_request, positions, out,
                                   n_tokens, nq, nkv, 1, hd, hd, page_size, page_stride, head_stride, page_stride, head_stride,
                                   scale, window, 0, dtype, 0, split_override, nullptr, stream);
}
