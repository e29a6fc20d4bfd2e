// Attention whose heads' scores are mixed before the softmax ("talking heads"):
//   s_g(i, j) = q_g(i) . k_kv(g)(j)            for every query head g (kv(g): its key/value head)
//   z_h(i, j) = sum_g mix[h][g] s_g(i, j)      a learned heads x heads matrix (score scale and a factor per head folded in)
//   p_h(i, :) = softmax over the visible keys of z_h(i, :)   (optionally with exp(sink_h) in the denominator)
//   o_h(i)    = sum_j p_h(i, j) v_kv(h)(j)     (optionally times sigmoid(gate[i, h]))
// A key is visible to a query at position p when it lies at p or before and, with a window, less than `window` back.
// The mixing makes every head's weights depend on all heads' scores, so one CTA takes ALL heads of a tile of QT
// consecutive queries of one request: warp g computes head g's scores against a staged tile of 32 keys (a lane per
// key; fewer keys where 32 of all key/value heads do not fit the shared memory), the scores meet in shared memory, warp h mixes its row of them, keeps the running maximum and denominator of
// its QT queries and adds the tile's weighted values (a lane per value column).  Scores, mixing, softmax and sums are
// 32-bit on the CUDA cores for both dtypes; keys and values are read from their pages in the cache's dtype.
#include "common.cuh"

TLLM_DEFINE_LAST_ERROR

namespace tllm {

constexpr int TK_MAX = 32;   // keys per staged tile: a lane per key; 16, 8 or 4 where larger tiles of all key/value heads do not fit

struct TalkArgs {
  const void* q;               // rows of ldq values; the first heads * kd are the query heads
  int ldq;
  const void *kcache, *vcache; // [pages, kv_heads, page_size, kd | vd]
  const int* block_table;      // [requests, max_blocks], -1: the page was given back
  int max_blocks;
  const int *cu_q, *q_start;
  const float* mix;            // [heads, heads]
  const float* sink;           // [heads] or null
  const void* gate;            // rows of ldg values, one per head, or null
  int ldg;
  void* out;                   // [T, heads * vd]
  int out_f32;
  int heads, kv_heads, kd, vd, page_size;
  long long k_page_stride, k_head_stride, v_page_stride, v_head_stride;
  int window;                  // 0: every earlier key
  int tk;                      // keys per staged tile
};

__host__ __device__ inline size_t talk_align(size_t x) { return (x + 15) & ~(size_t)15; }

// T: dtype of queries, cache and gate; QT: queries per CTA; VC: value columns per lane (32 * VC >= vd)
template <typename T, int QT, int VC>
__global__ void __launch_bounds__(QT * VC > 16 ? 512 : 1024) attention_talk_kernel(TalkArgs a) {
  extern __shared__ __align__(16) unsigned char smem[];
  pdl_trigger();
  const int H = a.heads, G = a.kv_heads, kd = a.kd, vd = a.vd, TK_KEYS = a.tk;
  const int ks = kd + 1;   // a key row's stride in shared memory: a lane per key reads without bank conflicts
  size_t at = 0;
  float* sq = reinterpret_cast<float*>(smem + at); at = talk_align(at + sizeof(float) * QT * H * kd);
  float* sk = reinterpret_cast<float*>(smem + at); at = talk_align(at + sizeof(float) * G * TK_KEYS * ks);
  float* ss = reinterpret_cast<float*>(smem + at); at = talk_align(at + sizeof(float) * H * QT * TK_KEYS);
  float* sp = reinterpret_cast<float*>(smem + at); at = talk_align(at + sizeof(float) * H * TK_KEYS * QT);
  float* smix = reinterpret_cast<float*>(smem + at); at = talk_align(at + sizeof(float) * H * H);
  T* sv = reinterpret_cast<T*>(smem + at);
  const int tid = threadIdx.x, nthreads = blockDim.x;
  const int h = tid >> 5, lane = tid & 31;
  for (int i = tid; i < H * H; i += nthreads) smix[i] = a.mix[i];   // constants of the model
  pdl_wait();
  const int r = blockIdx.y;
  const int first = a.cu_q[r], qlen = a.cu_q[r + 1] - first;
  const int i0 = blockIdx.x * QT;
  if (i0 >= qlen) return;
  const int nq = min(QT, qlen - i0);
  const int t0 = first + i0, p0 = a.q_start[r] + i0;
  const T* q = (const T*)a.q;
  for (int idx = tid; idx < QT * H * kd; idx += nthreads) {
    const int i = idx / (H * kd), rest = idx - i * (H * kd);
    sq[idx] = i < nq ? to_f32(q[(size_t)(t0 + i) * a.ldq + rest]) : 0.f;
  }
  const int* table = a.block_table + (size_t)r * a.max_blocks;
  const int kvh = h / (H / G);
  const int lo = a.window > 0 ? max(0, p0 - a.window + 1) : 0, hi = p0 + nq - 1;
  float m[QT], l[QT], acc[QT][VC];
#pragma unroll
  for (int i = 0; i < QT; ++i) {
    m[i] = -INFINITY; l[i] = 0.f;
#pragma unroll
    for (int c = 0; c < VC; ++c) acc[i][c] = 0.f;
  }
  const T* kc = (const T*)a.kcache;
  const T* vc = (const T*)a.vcache;
  // Key tiles begin at multiples of TK_KEYS whatever the tile of queries: a query then meets its keys in the same
  // tiles, lanes and order however its prompt was cut and whatever shares its CTA (a tile or a lane that it does not
  // see changes no bit of its sums), so the 32-bit results do not depend on the cut.
  for (int j0 = lo - lo % TK_KEYS; j0 <= hi; j0 += TK_KEYS) {
    const int nk = min(TK_KEYS, hi - j0 + 1);
    __syncthreads();   // the tile before is read to its end (and the queries are in place)
    for (int idx = tid; idx < G * TK_KEYS * kd; idx += nthreads) {
      const int g = idx / (TK_KEYS * kd), rest = idx - g * (TK_KEYS * kd), j = rest / kd, d = rest - j * kd;
      float x = 0.f;
      if (j < nk) {
        const int pos = j0 + j, page = table[pos / a.page_size];
        if (page >= 0) x = to_f32(kc[page * a.k_page_stride + g * a.k_head_stride + (long long)(pos % a.page_size) * kd + d]);
      }
      sk[(g * TK_KEYS + j) * ks + d] = x;
    }
    for (int idx = tid; idx < G * TK_KEYS * vd; idx += nthreads) {
      const int g = idx / (TK_KEYS * vd), rest = idx - g * (TK_KEYS * vd), j = rest / vd, d = rest - j * vd;
      T x = from_f32<T>(0.f);
      if (j < nk) {
        const int pos = j0 + j, page = table[pos / a.page_size];
        if (page >= 0) x = vc[page * a.v_page_stride + g * a.v_head_stride + (long long)(pos % a.page_size) * vd + d];
      }
      sv[idx] = x;
    }
    __syncthreads();
    {   // head h's scores of the tile: a lane per key, all QT queries at once so that a key value is read once
      float s[QT];
#pragma unroll
      for (int i = 0; i < QT; ++i) s[i] = 0.f;
      const float* kr = sk + (kvh * TK_KEYS + min(lane, TK_KEYS - 1)) * ks;
      const float* qr = sq + h * kd;
      if ((kd & 3) == 0) {
        for (int d = 0; d < kd; d += 4) {
          const float k0 = kr[d], k1 = kr[d + 1], k2 = kr[d + 2], k3 = kr[d + 3];
#pragma unroll
          for (int i = 0; i < QT; ++i) {
            const float4 qv = *reinterpret_cast<const float4*>(qr + (size_t)i * H * kd + d);
            s[i] = fmaf(qv.x, k0, s[i]); s[i] = fmaf(qv.y, k1, s[i]); s[i] = fmaf(qv.z, k2, s[i]); s[i] = fmaf(qv.w, k3, s[i]);
          }
        }
      } else {
        for (int d = 0; d < kd; ++d) {
          const float kv = kr[d];
#pragma unroll
          for (int i = 0; i < QT; ++i) s[i] = fmaf(qr[(size_t)i * H * kd + d], kv, s[i]);
        }
      }
#pragma unroll
      for (int i = 0; i < QT; ++i)
        if (lane < TK_KEYS) ss[(h * QT + i) * TK_KEYS + lane] = s[i];
    }
    __syncthreads();
    // head h's mixed scores, running maximum and denominator, and the tile's weights
    const int kpos = j0 + lane;
#pragma unroll
    for (int i = 0; i < QT; ++i) {
      float z = 0.f;
      if (lane < TK_KEYS)
        for (int g = 0; g < H; ++g) z = fmaf(smix[h * H + g], ss[(g * QT + i) * TK_KEYS + lane], z);
      const int qpos = p0 + i;
      const bool seen = i < nq && lane < nk && kpos <= qpos && (a.window <= 0 || qpos - kpos < a.window);
      z = seen ? z : -INFINITY;
      const float m_new = fmaxf(m[i], warp_max(z));
      const float alpha = m_new == -INFINITY ? 1.f : expf(m[i] - m_new);
      const float p = seen ? expf(z - m_new) : 0.f;
      l[i] = fmaf(l[i], alpha, warp_sum(p));
      m[i] = m_new;
#pragma unroll
      for (int c = 0; c < VC; ++c) acc[i][c] *= alpha;
      if (lane < TK_KEYS) sp[(h * TK_KEYS + lane) * QT + i] = p;
    }
    __syncwarp();
    const T* vr = sv + (size_t)kvh * TK_KEYS * vd;
    for (int j = 0; j < nk; ++j) {
      float pj[QT];
#pragma unroll
      for (int i = 0; i < QT; ++i) pj[i] = sp[(h * TK_KEYS + j) * QT + i];
#pragma unroll
      for (int c = 0; c < VC; ++c) {
        const int d = lane + 32 * c;
        if (d < vd) {
          const float vv = to_f32(vr[j * vd + d]);
#pragma unroll
          for (int i = 0; i < QT; ++i) acc[i][c] = fmaf(pj[i], vv, acc[i][c]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < QT; ++i) {
    if (i >= nq) break;
    float denom = l[i], keep = 1.f;
    if (a.sink) {   // exp(sink) joins the denominator, under a maximum that covers it
      const float sk_h = a.sink[h], m_f = fmaxf(m[i], sk_h);
      keep = expf(m[i] - m_f);
      denom = fmaf(l[i], keep, expf(sk_h - m_f));
    }
    float f = keep / denom;
    if (a.gate) {
      const float gv = to_f32(((const T*)a.gate)[(size_t)(t0 + i) * a.ldg + h]);
      f = f / (1.f + expf(-gv));
    }
    const size_t row = (size_t)(t0 + i) * H * vd + (size_t)h * vd;
#pragma unroll
    for (int c = 0; c < VC; ++c) {
      const int d = lane + 32 * c;
      if (d < vd) {
        const float y = __fmul_rn(acc[i][c], f);
        if (a.out_f32) ((float*)a.out)[row + d] = y;
        else ((T*)a.out)[row + d] = from_f32<T>(y);
      }
    }
  }
}

inline size_t talk_smem(int qt, int TK_KEYS, int heads, int kv_heads, int kd, int vd, size_t elem) {
  size_t at = 0;
  at = talk_align(at + sizeof(float) * qt * heads * kd);
  at = talk_align(at + sizeof(float) * kv_heads * TK_KEYS * (kd + 1));
  at = talk_align(at + sizeof(float) * heads * qt * TK_KEYS);
  at = talk_align(at + sizeof(float) * heads * TK_KEYS * qt);
  at = talk_align(at + sizeof(float) * heads * heads);
  return at + elem * kv_heads * TK_KEYS * vd;
}

template <typename T, int QT, int VC>
int talk_launch(const TalkArgs& a, int n_requests, int max_q_len, size_t smem, cudaStream_t s) {
  auto kernel = attention_talk_kernel<T, QT, VC>;
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      TLLM_FAIL(TLLM_ERR_CUDA, "attention_talk: %zu bytes of shared memory were refused", smem);
    configured = smem;
  }
  const dim3 grid((max_q_len + QT - 1) / QT, n_requests);
  TLLM_LAUNCH("attention_talk", kernel, grid, 32 * a.heads, smem, s, a);
  return TLLM_OK;
}

template <typename T, int QT>
int talk_pick_vc(const TalkArgs& a, int n_requests, int max_q_len, size_t smem, cudaStream_t s) {
  if (a.vd <= 32) return talk_launch<T, QT, 1>(a, n_requests, max_q_len, smem, s);
  if (a.vd <= 64) return talk_launch<T, QT, 2>(a, n_requests, max_q_len, smem, s);
  if (a.vd <= 128) return talk_launch<T, QT, 4>(a, n_requests, max_q_len, smem, s);
  return talk_launch<T, QT, 8>(a, n_requests, max_q_len, smem, s);
}

template <typename T>
int talk_pick(TalkArgs a, int n_requests, int max_q_len, cudaStream_t s) {
  constexpr size_t LIMIT = 200 * 1024;
  // as many queries per CTA as the shared memory holds (a key tile is staged once for all of them); one for decoding
  // The keys per tile depend on the model's sizes alone (never on the step), so that a query meets its keys in the
  // same tiles whatever the step looks like.
  int tk = TK_MAX;
  while (tk > 4 && talk_smem(1, tk, a.heads, a.kv_heads, a.kd, a.vd, sizeof(T)) > LIMIT) tk >>= 1;
  int qt = max_q_len >= 8 ? 8 : (max_q_len >= 4 ? 4 : (max_q_len >= 2 ? 2 : 1));
  while (qt > 1 && talk_smem(qt, tk, a.heads, a.kv_heads, a.kd, a.vd, sizeof(T)) > LIMIT) qt >>= 1;
  // more than 16 heads are more than 512 threads, which leaves a thread 64 registers: fewer sums per thread then
  const int vc = a.vd <= 32 ? 1 : (a.vd <= 64 ? 2 : (a.vd <= 128 ? 4 : 8));
  while (a.heads > 16 && qt > 1 && qt * vc > 16) qt >>= 1;
  TLLM_REQUIRE(a.heads <= 16 || qt * vc <= 16, "attention_talk: %d heads with values of %d (more than 16 heads take values of at most 128)", a.heads, a.vd);
  const size_t smem = talk_smem(qt, tk, a.heads, a.kv_heads, a.kd, a.vd, sizeof(T));
  TLLM_REQUIRE(smem <= LIMIT, "attention_talk: %d heads over %d key/value heads of %d / %d values need %zu bytes of shared memory",
               a.heads, a.kv_heads, a.kd, a.vd, smem);
  a.tk = tk;
  if (qt == 8) return talk_pick_vc<T, 8>(a, n_requests, max_q_len, smem, s);
  if (qt == 4) return talk_pick_vc<T, 4>(a, n_requests, max_q_len, smem, s);
  if (qt == 2) return talk_pick_vc<T, 2>(a, n_requests, max_q_len, smem, s);
  return talk_pick_vc<T, 1>(a, n_requests, max_q_len, smem, s);
}

}  // namespace tllm

using namespace tllm;

extern "C" int tllm_attention_talk(const void* q, int ldq, const void* kcache, const void* vcache, const int* block_table,
                                   int max_blocks, const int* cu_q, const int* q_start, const float* mix, const float* sink,
                                   const void* gate, int ldg, void* out, int out_f32, int n_requests, int max_q_len,
                                   int heads, int kv_heads, int kd, int vd, int page_size, long long k_page_stride,
                                   long long k_head_stride, long long v_page_stride, long long v_head_stride, int window,
                                   int dtype, void* stream) {
  TLLM_REQUIRE(n_requests > 0 && n_requests <= 65535 && max_q_len > 0 && heads > 0 && heads <= 32 && kv_heads > 0 &&
               heads % kv_heads == 0 && kd > 0 && vd > 0 && vd <= 256 && page_size > 0 && window >= 0,
               "attention_talk: %d requests, %d heads (at most 32) over %d key/value heads, sizes %d / %d (values at most 256)",
               n_requests, heads, kv_heads, kd, vd);
  TalkArgs a;
  a.q = q; a.ldq = ldq; a.kcache = kcache; a.vcache = vcache; a.block_table = block_table; a.max_blocks = max_blocks;
  a.cu_q = cu_q; a.q_start = q_start; a.mix = mix; a.sink = sink; a.gate = gate; a.ldg = ldg; a.out = out; a.out_f32 = out_f32;
  a.heads = heads; a.kv_heads = kv_heads; a.kd = kd; a.vd = vd; a.page_size = page_size; a.k_page_stride = k_page_stride;
  a.k_head_stride = k_head_stride; a.v_page_stride = v_page_stride; a.v_head_stride = v_head_stride; a.window = window;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TLLM_F32) return talk_pick<float>(a, n_requests, max_q_len, s);
  if (dtype == TLLM_BF16) return talk_pick<__nv_bfloat16>(a, n_requests, max_q_len, s);
  TLLM_FAIL(TLLM_ERR_ARG, "attention_talk: unknown dtype code %d", dtype);
}
