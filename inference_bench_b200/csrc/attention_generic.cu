// Generic attention kernels: any head size (even, up to 256), any number of heads and groups, any
// page size; float32 or bfloat16 storage with float32 arithmetic. They serve the float32 path of
// the whole model and every bfloat16 shape that has no tensor-core specialisation.
//
//  * qk_norm_rope_kv: sums the split-K partials of the qkv projection, applies the per-head RMSNorm
//    to q and k, rotates them, writes q out and k/v into the paged cache
//    (reference: crates/kir/src/cuda/attention/common.rs:49-96, rope.rs:13-23).
//  * attention_generic: one warp per (token, query head); online softmax over the keys that the
//    token may see (causal, optional window), read through the block table. Prefill portions and
//    decoded tokens are the same case here: a token at position p reads keys lo..p
//    (mask: crates/kir/src/cuda/attention/flash_mma.rs:193).
#include <type_traits>

#include "kv_view.cuh"

namespace {

constexpr int kWarps = 4;
constexpr int kMaxHeadDim = 256;

template <typename A, typename C>
__global__ void qk_norm_rope_kv_kernel(const float* __restrict__ qkv, int P, size_t stride_p, const float* __restrict__ q_norm_w,
                                       const float* __restrict__ k_norm_w, float eps, const float* __restrict__ cos_t,
                                       const float* __restrict__ sin_t, int rot_half, const int* __restrict__ positions,
                                       const int* __restrict__ seg_of_token, A* __restrict__ q_out, IbKvView kv, int write_kv, int T,
                                       int heads, unsigned* __restrict__ status, const float* __restrict__ bias, int qk_dim, int v_dim, int row, int q_col,
                                       int k_col, int v_col, int unit_norm_after) {
  // qk_dim, v_dim: sizes of a query/key head and of a value head (both at most the cache's row, kv.head_dim); the projection's row is
  // [heads x qk_dim | kv_heads x qk_dim | kv_heads x v_dim]. bias: one value per entry of that row, or null.
  // row > 0: the projection's row has `row` entries and the three parts start at q_col, k_col, v_col; v_col < 0: the values are the keys
  // as projected (with their bias, before any norm or rotation). unit_norm_after: q and k are divided by their root mean square over
  // the head after the rotation, without weights (q_norm_w and k_norm_w are then not read).
  __shared__ float vec[kWarps][kMaxHeadDim];
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int kvh = kv.kv_heads;
  const int slots = heads + 2 * kvh;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  long long item = (long long)blockIdx.x * kWarps + warp;
  if (item >= (long long)T * slots) return;
  const int t = (int)(item / slots), j = (int)(item % slots);
  const int R = row > 0 ? row : (heads + kvh) * qk_dim + kvh * v_dim;
  const bool is_q = j < heads, is_k = !is_q && j < heads + kvh;
  if (!is_q && !write_kv) return;
  const int hd = (is_q || is_k) ? qk_dim : v_dim;
  int col0 = (is_q || is_k) ? j * qk_dim : (heads + kvh) * qk_dim + (j - heads - kvh) * v_dim;
  if (row > 0) col0 = is_q ? q_col + j * qk_dim : (is_k ? k_col + (j - heads) * qk_dim : (v_col < 0 ? k_col + (j - heads - kvh) * qk_dim : v_col + (j - heads - kvh) * v_dim));
  const float* src = qkv + (size_t)t * R + col0;
  float* v = vec[warp];
  float ss = 0.f;
  for (int d = lane; d < hd; d += 32) {
    float a = src[d];
    for (int p = 1; p < P; p++) a += src[p * stride_p + d];
    if (bias) a += bias[col0 + d];
    v[d] = a;
    ss += a * a;
  }
  __syncwarp();
  const float* nw = unit_norm_after ? nullptr : (is_q ? q_norm_w : (is_k ? k_norm_w : nullptr));
  if (nw) {
    ss = ib::warp_sum(ss);
    float inv = rsqrtf(ss / (float)hd + eps);
    for (int d = lane; d < hd; d += 32) v[d] = nw[d] * (v[d] * inv);
    __syncwarp();
  }
  if ((is_q || is_k) && cos_t && rot_half > 0) {
    // Half rotation over the first 2*rot_half dims: pair (d, d + rot_half).
    for (int d = lane; d < rot_half; d += 32) {
      float c = cos_t[(size_t)t * rot_half + d], s = sin_t[(size_t)t * rot_half + d];
      float a = v[d], b = v[d + rot_half];
      v[d] = a * c - b * s;
      v[d + rot_half] = b * c + a * s;
    }
    __syncwarp();
  }
  if ((is_q || is_k) && unit_norm_after) {
    float s2 = 0.f;
    for (int d = lane; d < hd; d += 32) s2 = __fmaf_rn(v[d], v[d], s2);
    s2 = ib::warp_sum(s2);
    const float inv = 1.f / sqrtf(s2 / (float)hd + eps);
    for (int d = lane; d < hd; d += 32) v[d] *= inv;
    __syncwarp();
  }
  if (is_q) {
    A* dst = q_out + (size_t)t * heads * hd + (size_t)j * hd;
    for (int d = lane; d < hd; d += 32) dst[d] = ib::from_f32<A>(v[d]);
    return;
  }
  const int head = is_k ? j - heads : j - heads - kvh;
  long long off = ib::kv_offset(kv, seg_of_token[t], positions[t], head);
  if (off < 0) {
    if (lane == 0) atomicOr(status, IB_ERR_BAD_PAGE);
    return;
  }
  C* dst = (C*)kv.base + off + (is_k ? 0 : kv.v_offset);
  for (int d = lane; d < hd; d += 32) dst[d] = ib::from_f32<C>(v[d]);
}

// The same for head sizes 64 and 128 with the whole head rotated (or none of it): a lane holds
// HD/32 consecutive values, so loads and stores are 8 or 16 bytes wide, the norm is one warp sum,
// and the rotation partner (d + HD/2) sits in lane ^ 16.
template <int HD, typename A, typename C, int PER>
__global__ void qk_norm_rope_kv_vec_kernel(const float* __restrict__ qkv, int P, size_t stride_p, const float* __restrict__ q_norm_w,
                                           const float* __restrict__ k_norm_w, float eps, const float* __restrict__ cos_t,
                                           const float* __restrict__ sin_t, const int* __restrict__ positions,
                                           const int* __restrict__ seg_of_token, A* __restrict__ q_out, IbKvView kv, int write_kv, int T,
                                           int heads, unsigned* __restrict__ status, const float* __restrict__ bias) {
  // blockIdx.x is the token; a warp takes PER consecutive heads of it (q heads, then k heads, then v heads)
  // and loads them all before it works on any: with many tokens (PER = 4) that keeps four loads per lane
  // in flight; with few, PER = 1 keeps the chain short. No division anywhere: this kernel is bound by
  // its instruction count as much as by memory.
  constexpr int E = HD / 32;
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int kvh = kv.kv_heads, slots = heads + 2 * kvh;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int j0 = (blockIdx.y * kWarps + warp) * PER;
  // what every head of the token shares, fetched once per warp with wide loads and requested before the partial products
  // (one trip to memory for all of it, not one after the other): norm scales, the token's
  // rotation (the sine with the sign of this lane's half: d < HD/2: v cos - partner sin; d >= HD/2: v cos + partner sin)
  float qw[E], kw[E], cs[E], sn[E];
  auto load_vec = [&](const float* src, float (&dst)[E]) {
    if constexpr (E == 4) {
      const float4 a = *(const float4*)src;
      dst[0] = a.x, dst[1] = a.y, dst[2] = a.z, dst[3] = a.w;
    } else {
      const float2 a = *(const float2*)src;
      dst[0] = a.x, dst[1] = a.y;
    }
  };
  if (q_norm_w) load_vec(q_norm_w + lane * E, qw);
  if (k_norm_w) load_vec(k_norm_w + lane * E, kw);
  if (cos_t) {
    load_vec(cos_t + (size_t)t * (HD / 2) + (lane & 15) * E, cs);
    load_vec(sin_t + (size_t)t * (HD / 2) + (lane & 15) * E, sn);
  }
  float v[PER][E];
#pragma unroll
  for (int u = 0; u < PER; u++) {
#pragma unroll
    for (int e = 0; e < E; e++) v[u][e] = 0.f;
    const int j = j0 + u;
    if (j >= slots || (j >= heads && !write_kv)) continue;
    const float* src = qkv + (size_t)t * slots * HD + (size_t)j * HD + lane * E;
    for (int p = 0; p < P; p++) {
      if constexpr (E == 4) {
        const float4 a = *(const float4*)(src + p * stride_p);
        v[u][0] += a.x, v[u][1] += a.y, v[u][2] += a.z, v[u][3] += a.w;
      } else {
        const float2 a = *(const float2*)(src + p * stride_p);
        v[u][0] += a.x, v[u][1] += a.y;
      }
    }
    if (bias) {
#pragma unroll
      for (int e = 0; e < E; e++) v[u][e] += bias[(size_t)j * HD + lane * E + e];
    }
  }
  if (cos_t && lane < 16) {   // (used only now, so that nothing waited for it above)
#pragma unroll
    for (int e = 0; e < E; e++) sn[e] = -sn[e];
  }
#pragma unroll
  for (int u = 0; u < PER; u++) {
    const int j = j0 + u;
    if (j >= slots) continue;
    const bool is_q = j < heads, is_k = !is_q && j < heads + kvh;
    if (!is_q && !write_kv) continue;
    if (is_q ? q_norm_w != nullptr : (is_k && k_norm_w != nullptr)) {
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < E; e++) ss += v[u][e] * v[u][e];
      ss = ib::warp_sum(ss);
      const float inv = rsqrtf(ss / (float)HD + eps);
#pragma unroll
      for (int e = 0; e < E; e++) v[u][e] = (is_q ? qw[e] : kw[e]) * (v[u][e] * inv);
    }
    if ((is_q || is_k) && cos_t) {
#pragma unroll
      for (int e = 0; e < E; e++) {
        const float other = __shfl_xor_sync(0xffffffffu, v[u][e], 16);
        v[u][e] = __fmaf_rn(other, sn[e], __fmul_rn(v[u][e], cs[e]));
      }
    }
    auto store = [&](auto* dst) {
      using D = std::remove_pointer_t<decltype(dst)>;
      if constexpr (sizeof(D) == 4) {
        if constexpr (E == 4) *(float4*)dst = make_float4(v[u][0], v[u][1], v[u][2], v[u][3]);
        else *(float2*)dst = make_float2(v[u][0], v[u][1]);
      } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(v[u][0], v[u][1]);
        if constexpr (E == 4) {
          __nv_bfloat162 hi = __floats2bfloat162_rn(v[u][2], v[u][3]);
          *(uint2*)dst = make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
        } else {
          *(uint32_t*)dst = *(uint32_t*)&lo;
        }
      }
    };
    if (is_q) {
      store(q_out + (size_t)t * heads * HD + (size_t)j * HD + lane * E);
      continue;
    }
    const int head = is_k ? j - heads : j - heads - kvh;
    const long long off = ib::kv_offset(kv, seg_of_token[t], positions[t], head);
    if (off < 0) {
      if (lane == 0) atomicOr(status, IB_ERR_BAD_PAGE);
      continue;
    }
    store((C*)kv.base + off + (is_k ? 0 : kv.v_offset) + lane * E);
  }
}

// acc registers: lane owns dims lane, lane+32, ... (up to 8 for head_dim 256).
template <typename A, typename C>
__global__ void attention_generic_kernel(const A* __restrict__ q, IbKvView kv, const int* __restrict__ positions,
                                         const int* __restrict__ seg_of_token, int window, float scale, A* __restrict__ out, int T,
                                         int heads, unsigned* __restrict__ status, int qk_dim, int v_dim, float softcap, int sink, int chunk,
                                         const float* __restrict__ sink_values, const float* __restrict__ gate, int gate_P, size_t gate_stride, int gate_row,
                                         float out_scale, int out_row) {
  // qk_dim, v_dim: a query/key head's and a value head's size (at most the cache's row). softcap > 0: s <- softcap * tanh(s / softcap).
  // sink: the softmax has one more term whose score is 0 and which has no value (its denominator is 1 + sum exp(s)); with sink_values
  // the term's score is sink_values[head] instead (not scaled). chunk > 0: a position sees the earlier positions of its own block of
  // `chunk` positions, counted from position 0 (window is then not read). gate: float32 partial sums [gate_P][T][gate_row], offset to
  // the first head's column: head h's output is multiplied by sigmoid(gate[t][h]). out_scale multiplies every output; out_row: entries
  // of an output row (the heads' outputs are its first heads * v_dim).
  __shared__ float qs[kWarps][kMaxHeadDim];
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int hd = qk_dim, row = kv.head_dim;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  long long item = (long long)blockIdx.x * kWarps + warp;
  if (item >= (long long)T * heads) return;
  const int t = (int)(item / heads), h = (int)(item % heads);
  const int kvhead = h / (heads / kv.kv_heads);
  const int pos = positions[t], seg = seg_of_token[t];
  const int lo = chunk > 0 ? pos - pos % chunk : (window > 0 ? max(0, pos - window + 1) : 0);
  const A* qrow = q + (size_t)t * heads * hd + (size_t)h * hd;
  for (int d = lane; d < hd; d += 32) qs[warp][d] = ib::to_f32<A>(qrow[d]);
  __syncwarp();
  float acc[kMaxHeadDim / 32];
#pragma unroll
  for (int r = 0; r < kMaxHeadDim / 32; r++) acc[r] = 0.f;
  float m = sink ? (sink_values ? sink_values[h] : 0.f) : -INFINITY, l = sink ? 1.f : 0.f;   // the sink is a key of its own score: it starts the running maximum and sum
  (void)row;
  const C* base = (const C*)kv.base;
  for (int k0 = lo; k0 <= pos; k0 += 32) {
    int key = k0 + lane;
    long long off = -1;
    float s = -INFINITY;
    if (key <= pos) {
      off = ib::kv_offset(kv, seg, key, kvhead);
      if (off < 0) {
        atomicOr(status, IB_ERR_BAD_PAGE);
      } else {
        const C* kr = base + off;
        float dot = 0.f;
        for (int d = 0; d < hd; d++) dot += qs[warp][d] * ib::to_f32<C>(kr[d]);
        s = dot * scale;
        if (softcap > 0.f) s = softcap * tanhf(s / softcap);
      }
    }
    float m_new = fmaxf(m, ib::warp_max(s));
    if (m_new == -INFINITY) continue;  // every key of this chunk was unreadable
    float corr = expf(m - m_new);
    float p = s == -INFINITY ? 0.f : expf(s - m_new);
    l = l * corr + ib::warp_sum(p);
#pragma unroll
    for (int r = 0; r < kMaxHeadDim / 32; r++) acc[r] *= corr;
    int n = min(32, pos - k0 + 1);
    for (int jj = 0; jj < n; jj++) {
      float pj = __shfl_sync(0xffffffffu, p, jj);
      long long oj = __shfl_sync(0xffffffffu, off, jj);
      if (oj < 0) continue;
      const C* vr = base + oj + kv.v_offset;
#pragma unroll
      for (int r = 0; r < kMaxHeadDim / 32; r++) {
        int d = lane + 32 * r;
        if (d < v_dim) acc[r] += pj * ib::to_f32<C>(vr[d]);
      }
    }
    m = m_new;
  }
  float inv = (l > 0.f ? 1.f / l : 0.f) * out_scale;
  if (gate) {
    const float* gr = gate + (size_t)t * gate_row + h;
    float g = gr[0];
    for (int p = 1; p < gate_P; p++) g += gr[p * gate_stride];
    inv *= 1.f / (1.f + expf(-g));
  }
  A* orow = out + (size_t)t * out_row + (size_t)h * v_dim;
#pragma unroll
  for (int r = 0; r < kMaxHeadDim / 32; r++) {
    int d = lane + 32 * r;
    if (d < v_dim) orow[d] = ib::from_f32<A>(acc[r] * inv);
  }
}

int check_view(const char* name, const IbKvView* kv, int heads) {
  IB_CHECK_ARG(kv && kv->base && kv->block_table, "%s: the cache view has a null pointer", name);
  IB_CHECK_ARG(kv->head_dim > 0 && kv->head_dim <= kMaxHeadDim && kv->head_dim % 2 == 0,
               "%s: head_dim %d is not supported (even sizes up to %d)", name, kv->head_dim, kMaxHeadDim);
  IB_CHECK_ARG(kv->kv_heads > 0 && heads > 0 && heads % kv->kv_heads == 0, "%s: %d query heads are not a multiple of %d kv heads", name,
               heads, kv->kv_heads);
  IB_CHECK_ARG(kv->page_size > 0 && kv->num_pages > 0 && kv->table_stride > 0, "%s: bad page geometry", name);
  IB_CHECK_ARG(kv->dtype == IB_F32 || kv->dtype == IB_BF16, "%s: unknown cache dtype %d", name, kv->dtype);
  return 0;
}

}  // namespace

extern "C" int ib_qk_norm_rope_kv(const float* qkv, int P, long long stride_p, const float* q_norm_w, const float* k_norm_w, float eps,
                                  const float* cos_t, const float* sin_t, int rot_half, const int* positions, const int* seg_of_token,
                                  void* q_out, int act_dtype, const IbKvView* kv, int write_kv, int T, int heads, unsigned* status,
                                  const float* bias, int qk_dim, int v_dim, int row, int q_col, int k_col, int v_col, int unit_norm_after, cudaStream_t stream) {
  // qk_dim, v_dim: 0 = the cache's row size. bias: float32, one value per column of the projection, or null.
  // row, q_col, k_col, v_col, unit_norm_after: see the kernel; row = 0 stands for the row [q | k | v] alone.
  if (T == 0) return 0;
  if (check_view("qk_norm_rope_kv", kv, heads)) return 1;
  if (qk_dim <= 0) qk_dim = kv->head_dim;
  if (v_dim <= 0) v_dim = kv->head_dim;
  IB_CHECK_ARG(P >= 1 && T > 0, "qk_norm_rope_kv: bad sizes T=%d P=%d", T, P);
  IB_CHECK_ARG(qk_dim <= kv->head_dim && v_dim <= kv->head_dim, "qk_norm_rope_kv: head sizes %d and %d exceed the cache's row of %d", qk_dim, v_dim, kv->head_dim);
  IB_CHECK_ARG(rot_half >= 0 && 2 * rot_half <= qk_dim, "qk_norm_rope_kv: rotary size %d exceeds head_dim %d", 2 * rot_half, qk_dim);
  IB_CHECK_ARG((act_dtype == IB_F32 && kv->dtype == IB_F32) || (act_dtype == IB_BF16 && kv->dtype == IB_BF16),
               "qk_norm_rope_kv: activation dtype %d and cache dtype %d must match", act_dtype, kv->dtype);
  long long items = (long long)T * (heads + 2 * kv->kv_heads);
  unsigned blocks = (unsigned)((items + kWarps - 1) / kWarps);
  const int hd = kv->head_dim;
  const bool aligned = ((uintptr_t)qkv % 16 == 0) && (stride_p % 4 == 0) && ((uintptr_t)q_out % 16 == 0) && ((uintptr_t)kv->base % 16 == 0);
  IB_CHECK_ARG(row == 0 || (q_col >= 0 && k_col >= 0 && q_col + heads * qk_dim <= row && k_col + kv->kv_heads * qk_dim <= row && (v_col < 0 ? v_dim == qk_dim : v_col + kv->kv_heads * v_dim <= row)),
               "qk_norm_rope_kv: the parts at %d, %d, %d do not fit a row of %d (values that are the keys need the keys' size)", q_col, k_col, v_col, row);
  const bool vec = row == 0 && !unit_norm_after && (hd == 64 || hd == 128) && qk_dim == hd && v_dim == hd && (rot_half == 0 || 2 * rot_half == hd) && aligned;
  const float* cs = rot_half ? cos_t : nullptr;
  if (vec) {
    const int slots = heads + 2 * kv->kv_heads;
    auto go = [&](auto kernel, int per, auto* qo) {
      const dim3 grid((unsigned)T, (unsigned)((slots + kWarps * per - 1) / (kWarps * per)));
      ib::launch(kernel, grid, kWarps * 32, 0, stream, qkv, P, (size_t)stride_p, q_norm_w, k_norm_w, eps, cs, sin_t, positions, seg_of_token, qo, *kv,
                 write_kv, T, heads, status, bias);
    };
    const bool many = (long long)T * slots >= 8192;   // a prompt portion: four heads per warp; a few decoded tokens: one
    if (act_dtype == IB_F32 && hd == 128) {
      if (many) go(qk_norm_rope_kv_vec_kernel<128, float, float, 4>, 4, (float*)q_out);
      else go(qk_norm_rope_kv_vec_kernel<128, float, float, 1>, 1, (float*)q_out);
    } else if (act_dtype == IB_F32) {
      if (many) go(qk_norm_rope_kv_vec_kernel<64, float, float, 4>, 4, (float*)q_out);
      else go(qk_norm_rope_kv_vec_kernel<64, float, float, 1>, 1, (float*)q_out);
    } else if (hd == 128) {
      if (many) go(qk_norm_rope_kv_vec_kernel<128, __nv_bfloat16, __nv_bfloat16, 4>, 4, (__nv_bfloat16*)q_out);
      else go(qk_norm_rope_kv_vec_kernel<128, __nv_bfloat16, __nv_bfloat16, 1>, 1, (__nv_bfloat16*)q_out);
    } else {
      if (many) go(qk_norm_rope_kv_vec_kernel<64, __nv_bfloat16, __nv_bfloat16, 4>, 4, (__nv_bfloat16*)q_out);
      else go(qk_norm_rope_kv_vec_kernel<64, __nv_bfloat16, __nv_bfloat16, 1>, 1, (__nv_bfloat16*)q_out);
    }
  }
  else if (act_dtype == IB_F32)
    ib::launch(qk_norm_rope_kv_kernel<float, float>, blocks, kWarps * 32, 0, stream, qkv, P, (size_t)stride_p, q_norm_w, k_norm_w, eps, cos_t, sin_t,
                                                                            rot_half, positions, seg_of_token, (float*)q_out, *kv, write_kv,
                                                                            T, heads, status, bias, qk_dim, v_dim, row, q_col, k_col, v_col, unit_norm_after);
  else
    ib::launch(qk_norm_rope_kv_kernel<__nv_bfloat16, __nv_bfloat16>, blocks, kWarps * 32, 0, stream, 
        qkv, P, (size_t)stride_p, q_norm_w, k_norm_w, eps, cos_t, sin_t, rot_half, positions, seg_of_token, (__nv_bfloat16*)q_out, *kv,
        write_kv, T, heads, status, bias, qk_dim, v_dim, row, q_col, k_col, v_col, unit_norm_after);
  IB_CHECK_LAUNCH("qk_norm_rope_kv");
  return 0;
}

extern "C" int ib_attention_generic(const void* q, int act_dtype, const IbKvView* kv, const int* positions, const int* seg_of_token,
                                    int window, float scale, void* out, int T, int heads, unsigned* status, int qk_dim, int v_dim, float softcap, int sink,
                                    int chunk, const float* sink_values, const float* gate, int gate_P, long long gate_stride, int gate_row, float out_scale,
                                    int out_row, cudaStream_t stream) {
  // chunk, sink_values, gate, out_scale, out_row: see the kernel; out_row = 0 stands for heads * v_dim, gate = null for no gate.
  // qk_dim, v_dim: 0 = the cache's row size; softcap: 0 = scores as they are; sink: 1 = one added to the softmax's denominator.
  if (T == 0) return 0;
  if (check_view("attention_generic", kv, heads)) return 1;
  if (qk_dim <= 0) qk_dim = kv->head_dim;
  if (v_dim <= 0) v_dim = kv->head_dim;
  IB_CHECK_ARG(qk_dim <= kv->head_dim && v_dim <= kv->head_dim, "attention_generic: head sizes %d and %d exceed the cache's row of %d", qk_dim, v_dim, kv->head_dim);
  IB_CHECK_ARG((act_dtype == IB_F32 && kv->dtype == IB_F32) || (act_dtype == IB_BF16 && kv->dtype == IB_BF16),
               "attention_generic: activation dtype %d and cache dtype %d must match", act_dtype, kv->dtype);
  if (out_row <= 0) out_row = heads * v_dim;
  IB_CHECK_ARG(out_row >= heads * v_dim && chunk >= 0 && (!sink_values || sink), "attention_generic: bad output row %d, chunk %d or sink values without a sink", out_row, chunk);
  long long items = (long long)T * heads;
  unsigned blocks = (unsigned)((items + kWarps - 1) / kWarps);
  if (act_dtype == IB_F32)
    ib::launch(attention_generic_kernel<float, float>, blocks, kWarps * 32, 0, stream, (const float*)q, *kv, positions, seg_of_token, window, scale,
                                                                              (float*)out, T, heads, status, qk_dim, v_dim, softcap, sink, chunk, sink_values, gate,
                                                                              gate_P, (size_t)gate_stride, gate_row, out_scale, out_row);
  else
    ib::launch(attention_generic_kernel<__nv_bfloat16, __nv_bfloat16>, blocks, kWarps * 32, 0, stream, 
        (const __nv_bfloat16*)q, *kv, positions, seg_of_token, window, scale, (__nv_bfloat16*)out, T, heads, status, qk_dim, v_dim, softcap, sink, chunk,
        sink_values, gate, gate_P, (size_t)gate_stride, gate_row, out_scale, out_row);
  IB_CHECK_LAUNCH("attention_generic");
  return 0;
}
