// Latent attention on the tensor cores, bfloat16: the same sum as latent_attention.cu's generic kernel
// (a head's query [Wuk^T q_n | q_r] against the cached rows [c | kr], softmax in float32, weighted sum of the latents c),
// for row sizes that are multiples of 16.
//
// A CTA of eight warps owns 16, 32 or 64 query rows: the heads of one token (blocks of heads when there are more; several consecutive
// tokens of one request when a prompt portion has them), and walks the keys they see in tiles of 64, which all its rows
// share: a cached row is read once for all of them (with 16 rows the kernel is bound by the key tiles' way from L2). Per tile:
//   S = Q K^T   warp w takes keys 8w..8w+7 over the whole row (m16n8k16, float32 accumulators), scales and masks them,
//               and the warps exchange row maxima and row sums through shared memory;
//   P           float32 weights exp(s - m), rounded to bfloat16 only as the operand of the second product; the sums l use
//               the float32 values;
//   O += P C    warp w takes the latent's 16-value chunks w, w + 8, ... of all 64 keys.
// Key tiles are copied with 16-byte cp.async through the block table into two swizzled buffers (the next tile arrives while
// this one is used); rows past the last visible key are zero-filled. With slices (steps of single decoded tokens), a CTA
// takes one slice of the keys and writes unnormalised partial results that latent_combine merges.
#include <type_traits>

#include "kv_view.cuh"
#include "mma_tiles.cuh"

namespace {

constexpr int kKeys = 64;    // keys of a tile
constexpr int kWarps = 8;
constexpr int kKeysPerWarp = kKeys / kWarps;   // 8: one n-tile of the S product a warp

// NCH: 16-value chunks of the latent a warp owns at most (rank <= 16 * kWarps * NCH). MT: 16-row tiles of queries a CTA holds.
template <int NCH, int MT>
__global__ void __launch_bounds__(kWarps * 32) latent_attention_mma_kernel(const float* __restrict__ q, IbKvView kv, const int* __restrict__ positions,
                                                                           const int* __restrict__ seg_of_token, const int2* __restrict__ units, float scale,
                                                                           __nv_bfloat16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                                                                           int H, int rank, int D, int n_slices, int slice_keys, unsigned* __restrict__ status,
                                                                           int window) {
  // window > 0: a token sees itself and the window - 1 positions before it; the CTA's keys start where its first token's window does.
  constexpr int R = 16 * MT;                                 // query rows of the CTA
  extern __shared__ __align__(128) unsigned char smem[];
  const int blocks = (D + 63) / 64;                          // 64-value blocks of a row
  const uint32_t k_bytes = (uint32_t)blocks * kKeys * 128;   // one key tile
  const uint32_t s_k = mt::smem_u32(smem);                   // two key tiles
  const uint32_t s_q = s_k + 2 * k_bytes;                    // [R][D]
  const uint32_t s_p = s_q + (uint32_t)blocks * R * 128;     // [R][64]
  float* wmax = (float*)(smem + 2 * k_bytes + (size_t)blocks * R * 128 + R * 128);   // [warps][R]
  float* wsum = wmax + kWarps * R;                                                   // [warps][R]
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
  const int hpc = H < R ? H : R;                             // heads a CTA covers
  const int h0 = blockIdx.x * hpc;
  // the last units first: in a prompt portion they see the most keys, and the short ones then fill the end of the launch
  const int ui = gridDim.y - 1 - blockIdx.y;
  int tok0 = ui, ntok = 1;
  if (units) {
    const int2 u = units[ui];
    tok0 = u.x, ntok = u.y;
  }
  const int slice = blockIdx.z;
  const int seg = seg_of_token[tok0];
  const int last_pos = positions[tok0 + ntok - 1];
  const int lo = (window > 0 ? max(0, positions[tok0] - window + 1) : 0) + slice * slice_keys;
  const int hi = min(last_pos, lo + slice_keys - 1);
  const int reach = window > 0 ? window : 0x7fffffff;   // a row at position p sees keys above p - reach
  // the rows this thread sees in its accumulators: g + 8 e of every 16-row tile
  int row_pos[MT][2], row_tok[MT][2], row_head[MT][2];
#pragma unroll
  for (int a = 0; a < MT; a++)
#pragma unroll
    for (int e = 0; e < 2; e++) {
      const int r = 16 * a + g + 8 * e, tl = r / hpc, hh = r - tl * hpc;
      const bool valid = tl < ntok && h0 + hh < H;
      row_tok[a][e] = valid ? tok0 + tl : -1;
      row_head[a][e] = h0 + hh;
      row_pos[a][e] = valid ? positions[tok0 + tl] : -1;
    }
  // queries -> bfloat16, swizzled [R][D]
  for (int idx = tid; idx < R * (D / 8); idx += kWarps * 32) {
    const int r = idx / (D / 8), c = idx - r * (D / 8);
    const int tl = r / hpc, hh = r - tl * hpc;
    uint32_t w[4] = {0u, 0u, 0u, 0u};
    if (tl < ntok && h0 + hh < H) {
      const float* src = q + ((size_t)(tok0 + tl) * H + h0 + hh) * D + c * 8;
      const float4 a = *(const float4*)src, b = *(const float4*)(src + 4);
      w[0] = mt::pack_bf16(a.x, a.y), w[1] = mt::pack_bf16(a.z, a.w), w[2] = mt::pack_bf16(b.x, b.y), w[3] = mt::pack_bf16(b.z, b.w);
    }
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(s_q + mt::tile_offset<64, R>(r, c)), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
  }
  const __nv_bfloat16* base = (const __nv_bfloat16*)kv.base;
  // eight threads copy one row's 128-byte pieces; 32 rows a pass. What a thread's addresses share is computed once: a warp is
  // alone on its scheduler here, and every instruction that is not a product or a copy is time.
  const int r7 = lane & 7;
  const uint32_t cp_off = (uint32_t)((tid >> 3) * 128 + (((tid & 7) ^ ((tid >> 3) & 7)) << 4));
  const int cp_iters = (D / 8 - (tid & 7) + 7) / 8;
  // The rows' places in the pool (a look-up in the block table each: a trip to memory) are fetched one tile ahead of the copies
  // that use them, so that no warp waits for them between a barrier and its products.
  constexpr int kPasses = kKeys / (kWarps * 4);
  long long off[kPasses];
  auto look_up = [&](int k0) {
#pragma unroll
    for (int pass = 0; pass < kPasses; pass++) {
      const int key = k0 + pass * (kWarps * 4) + (tid >> 3);
      off[pass] = -1;
      if (key <= hi) {
        off[pass] = ib::kv_offset(kv, seg, key, 0);
        if (off[pass] < 0) atomicOr(status, IB_ERR_BAD_PAGE);
      }
    }
  };
  auto issue_tile = [&](int buf) {   // the tile whose rows `off` holds
    const uint32_t dst = s_k + buf * k_bytes + cp_off;
#pragma unroll
    for (int pass = 0; pass < kPasses; pass++) {
      const __nv_bfloat16* src = base + off[pass] + (tid & 7) * 8;
      uint32_t at = dst + pass * (kWarps * 4 * 128);
      if (off[pass] >= 0) {
        for (int it = 0; it < cp_iters; it++, at += kKeys * 128, src += 64) mt::cp_async16(at, src);
      } else {
        for (int it = 0; it < cp_iters; it++, at += kKeys * 128) mt::st_shared_zero16(at);
      }
    }
    mt::cp_async_commit();
  };
  // fragment addresses: a fragment row's low three bits are the lane's, so the swizzle of the four 16-value steps of a 64-value block
  // is four constants a thread; a block further on is a fixed stride
  const int hb = lane >> 4, mb = (lane >> 3) & 1;
  const uint32_t a_row_off = (uint32_t)((r7 + 8 * mb) * 128);           // Q, P and V fragments: row (lane & 7) + 8 * ((lane >> 3) & 1) of their 16
  const uint32_t k_row_off = (uint32_t)((kKeysPerWarp * warp + r7) * 128);   // K fragments: this warp's 8 keys (lanes 0-15 give the addresses)
  uint32_t sw_a[4], sw_k[4];
#pragma unroll
  for (int j = 0; j < 4; j++) {
    sw_a[j] = (uint32_t)(((2 * j + hb) ^ r7) << 4);
    sw_k[j] = (uint32_t)(((2 * j + mb) ^ r7) << 4);
  }
  // V fragments: chunk 2 (warp + 8 i) + hb = block 2 i + (2 warp + hb) / 8, place (2 warp + hb) % 8
  const uint32_t v_off = a_row_off + (uint32_t)(((2 * warp + hb) >> 3) * kKeys * 128 + ((((2 * warp + hb) & 7) ^ r7) << 4));
  float o[MT][NCH][2][4];
  float m[MT][2], l[MT][2];
#pragma unroll
  for (int a = 0; a < MT; a++) {
    m[a][0] = m[a][1] = -INFINITY;
    l[a][0] = l[a][1] = 0.f;
#pragma unroll
    for (int i = 0; i < NCH; i++)
#pragma unroll
      for (int n = 0; n < 2; n++)
#pragma unroll
        for (int e = 0; e < 4; e++) o[a][i][n][e] = 0.f;
  }
  const int n_tiles = hi >= lo ? (hi - lo) / kKeys + 1 : 0;
  if (n_tiles > 0) {
    look_up(lo);
    issue_tile(0);
    if (n_tiles > 1) look_up(lo + kKeys);
  }
  for (int j = 0; j < n_tiles; j++) {
    const int k0 = lo + j * kKeys, buf = j & 1;
    mt::cp_async_wait<0>();
    __syncthreads();                                       // tile j is here; everybody is done with tile j - 1 and with P
    if (j + 1 < n_tiles) {
      issue_tile(buf ^ 1);
      if (j + 2 < n_tiles) look_up(k0 + 2 * kKeys);
    }
    const uint32_t kt = s_k + buf * k_bytes;
    // ---- S: this warp's 8 keys, every row tile
    float s[MT][4];
#pragma unroll
    for (int a = 0; a < MT; a++)
#pragma unroll
      for (int e = 0; e < 4; e++) s[a][e] = 0.f;
    {
      const int ksteps = D / 16;
      uint32_t ka = kt + k_row_off, qa = s_q + a_row_off;
      for (int kk0 = 0; kk0 < ksteps; kk0 += 4, ka += kKeys * 128, qa += R * 128) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
          if (kk0 + j < ksteps) {   // only the last block of a row may be partial
            uint32_t b0, b1, fa[MT][4];
            asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(ka + sw_k[j]));
#pragma unroll
            for (int a = 0; a < MT; a++) mt::ldmatrix_x4(qa + a * 2048 + sw_a[j], fa[a][0], fa[a][1], fa[a][2], fa[a][3]);
#pragma unroll
            for (int a = 0; a < MT; a++) mt::mma_16816(s[a], fa[a], b0, b1);
          }
        }
      }
    }
#pragma unroll
    for (int a = 0; a < MT; a++) {
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const int key = k0 + kKeysPerWarp * warp + 2 * t4 + (e & 1), rr = e >> 1;
        const float v = (key <= hi && key <= row_pos[a][rr] && row_pos[a][rr] - key < reach) ? s[a][e] * scale : -INFINITY;
        s[a][e] = v;
        mx[rr] = fmaxf(mx[rr], v);
      }
#pragma unroll
      for (int rr = 0; rr < 2; rr++) {
        mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
        mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
        if (t4 == 0) wmax[warp * R + 16 * a + g + 8 * rr] = mx[rr];
      }
    }
    __syncthreads();
    float corr[MT][2];
#pragma unroll
    for (int a = 0; a < MT; a++) {
      float sum[2];
#pragma unroll
      for (int rr = 0; rr < 2; rr++) {
        const int r = 16 * a + g + 8 * rr;
        float mt_ = wmax[r];
#pragma unroll
        for (int w = 1; w < kWarps; w++) mt_ = fmaxf(mt_, wmax[w * R + r]);
        const float m_new = fmaxf(m[a][rr], mt_);
        corr[a][rr] = m_new == -INFINITY ? 1.f : __expf(m[a][rr] - m_new);
        m[a][rr] = m_new;
        sum[rr] = 0.f;
      }
      float p[4];
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const int rr = e >> 1;
        p[e] = s[a][e] == -INFINITY ? 0.f : __expf(s[a][e] - m[a][rr]);
        sum[rr] += p[e];
      }
      // this warp's 8 keys are chunk `warp` of the P tile's 64
      asm volatile("st.shared.u32 [%0], %1;" ::"r"(s_p + mt::tile_offset<64, R>(16 * a + g, warp) + 4 * t4), "r"(mt::pack_bf16(p[0], p[1])) : "memory");
      asm volatile("st.shared.u32 [%0], %1;" ::"r"(s_p + mt::tile_offset<64, R>(16 * a + g + 8, warp) + 4 * t4), "r"(mt::pack_bf16(p[2], p[3])) : "memory");
#pragma unroll
      for (int rr = 0; rr < 2; rr++) {
        sum[rr] += __shfl_xor_sync(0xffffffffu, sum[rr], 1);
        sum[rr] += __shfl_xor_sync(0xffffffffu, sum[rr], 2);
        if (t4 == 0) wsum[warp * R + 16 * a + g + 8 * rr] = sum[rr];
      }
    }
    __syncthreads();
#pragma unroll
    for (int a = 0; a < MT; a++) {
#pragma unroll
      for (int rr = 0; rr < 2; rr++) {
        const int r = 16 * a + g + 8 * rr;
        float t = wsum[r];
#pragma unroll
        for (int w = 1; w < kWarps; w++) t += wsum[w * R + r];
        l[a][rr] = l[a][rr] * corr[a][rr] + t;
      }
#pragma unroll
      for (int i = 0; i < NCH; i++)
#pragma unroll
        for (int n = 0; n < 2; n++) {
          o[a][i][n][0] *= corr[a][0], o[a][i][n][1] *= corr[a][0];
          o[a][i][n][2] *= corr[a][1], o[a][i][n][3] *= corr[a][1];
        }
    }
    // ---- O += P C: this warp's chunks of the latent; the next chunk's fragment is requested before this one's products
#pragma unroll
    for (int ks = 0; ks < kKeys / 16; ks++) {
      uint32_t fa[MT][4];
#pragma unroll
      for (int a = 0; a < MT; a++) mt::ldmatrix_x4(s_p + a_row_off + a * 2048 + sw_a[ks], fa[a][0], fa[a][1], fa[a][2], fa[a][3]);
      const uint32_t va = kt + v_off + ks * 2048;
      uint32_t r[2][4];
      if (warp * 16 < rank) mt::ldmatrix_x4_trans(va, r[0][0], r[0][1], r[0][2], r[0][3]);
#pragma unroll
      for (int i = 0; i < NCH; i++) {
        const int dp = warp + kWarps * i;
        if (i + 1 < NCH && (dp + kWarps) * 16 < rank)
          mt::ldmatrix_x4_trans(va + (i + 1) * (kWarps / 4) * kKeys * 128, r[(i + 1) & 1][0], r[(i + 1) & 1][1], r[(i + 1) & 1][2], r[(i + 1) & 1][3]);
        if (dp * 16 < rank) {
#pragma unroll
          for (int a = 0; a < MT; a++) {
            mt::mma_16816(o[a][i][0], fa[a], r[i & 1][0], r[i & 1][1]);
            mt::mma_16816(o[a][i][1], fa[a], r[i & 1][2], r[i & 1][3]);
          }
        }
      }
    }
  }
  // ---- out
#pragma unroll
  for (int a = 0; a < MT; a++)
#pragma unroll
    for (int rr = 0; rr < 2; rr++) {
      if (row_tok[a][rr] < 0) continue;
      const size_t th = (size_t)row_tok[a][rr] * H + row_head[a][rr];
      if (n_slices == 1) {
        const float inv = l[a][rr] > 0.f ? 1.f / l[a][rr] : 0.f;
        __nv_bfloat16* dst = out + th * rank;
#pragma unroll
        for (int i = 0; i < NCH; i++) {
          const int dp = warp + kWarps * i;
          if (dp * 16 >= rank) continue;
#pragma unroll
          for (int n = 0; n < 2; n++)
            *(uint32_t*)(dst + dp * 16 + 8 * n + 2 * t4) = mt::pack_bf16(o[a][i][n][2 * rr] * inv, o[a][i][n][2 * rr + 1] * inv);
        }
      } else {
        const size_t unit = th * n_slices + slice;
        float* dst = part_o + unit * rank;
#pragma unroll
        for (int i = 0; i < NCH; i++) {
          const int dp = warp + kWarps * i;
          if (dp * 16 >= rank) continue;
#pragma unroll
          for (int n = 0; n < 2; n++) *(float2*)(dst + dp * 16 + 8 * n + 2 * t4) = make_float2(o[a][i][n][2 * rr], o[a][i][n][2 * rr + 1]);
        }
        if (warp == 0 && t4 == 0) {
          part_ml[2 * unit] = m[a][rr];
          part_ml[2 * unit + 1] = l[a][rr];
        }
      }
    }
}

size_t latent_mma_smem(int D, int mt) {
  const int blocks = (D + 63) / 64, R = 16 * mt;
  return (size_t)2 * blocks * kKeys * 128 + (size_t)blocks * R * 128 + (size_t)R * 128 + 2 * kWarps * R * sizeof(float);
}

}  // namespace

extern "C" int ib_latent_combine(const float* part_o, const float* part_ml, void* out, int out_dtype, int rows, int rank, int n_slices, cudaStream_t stream);

// 1 when the tensor-core kernel takes these sizes (bfloat16 cache rows of D values of which the first `rank` are the latent).
extern "C" int ib_latent_attention_mma_supports(int rank, int D) { return rank > 0 && rank % 16 == 0 && D % 16 == 0 && rank <= D && rank <= 512 && D <= 576; }

// How many query rows a CTA of the tensor-core kernel holds for these sizes when a step has `rows_wanted` rows that can share key tiles
// (the heads of a token, times the consecutive tokens of a prompt portion): 16, 32 or 64, bounded by registers (a latent above 256
// values: 32) and by shared memory (two key tiles, the queries and the weights must fit).
extern "C" int ib_latent_attention_mma_rows(int rank, int D, int rows_wanted) {
  int mt = rank > 256 ? 2 : 4;
  while (mt > 1 && (16 * (mt / 2) >= rows_wanted || latent_mma_smem(D, mt) > 200 * 1024)) mt /= 2;
  // two CTAs an SM beat one with twice the rows (measured: 8 heads of 256 + 32, 2,048 tokens: 154 against 197 us), where halving makes room for two
  if (mt > 1 && 16 * (mt / 2) < rows_wanted && latent_mma_smem(D, mt) > 110 * 1024 && latent_mma_smem(D, mt / 2) <= 110 * 1024) mt /= 2;
  return 16 * mt;
}

extern "C" int ib_latent_attention_mma(const float* q, const IbKvView* kv, const int* positions, const int* seg_of_token, const int* units, int n_units, int rows,
                                       float scale, void* out, float* part_o, float* part_ml, int T, int heads, int rank, int n_slices, int slice_keys,
                                       unsigned* status, int window, cudaStream_t stream) {
  if (T == 0 || n_units == 0) return 0;
  IB_CHECK_ARG(kv && kv->base && kv->block_table && kv->kv_heads == 1 && kv->dtype == IB_BF16, "latent_attention_mma: a bfloat16 cache of one row per token is needed");
  const int D = kv->head_dim;
  IB_CHECK_ARG(ib_latent_attention_mma_supports(rank, D), "latent_attention_mma: rank %d of a row of %d is not supported (multiples of 16, up to 512 of 576)", rank, D);
  IB_CHECK_ARG(heads > 0 && n_slices >= 1 && slice_keys >= 1 && (n_slices == 1 || slice_keys % kKeys == 0), "latent_attention_mma: bad slicing %d x %d", n_slices,
               slice_keys);
  IB_CHECK_ARG(n_slices == 1 || (part_o && part_ml), "latent_attention_mma: slices need scratch");
  IB_CHECK_ARG(n_units <= 65535 && n_slices <= 65535, "latent_attention_mma: %d units or %d slices exceed the grid limit", n_units, n_slices);
  IB_CHECK_ARG(((uintptr_t)q % 16 == 0) && ((uintptr_t)kv->base % 16 == 0) && (kv->page_stride % 8 == 0), "latent_attention_mma: pointers must be 16-byte aligned");
  IB_CHECK_ARG((rows == 16 || rows == 32 || rows == 64) && !(rows == 64 && rank > 256), "latent_attention_mma: %d query rows a CTA (16, 32, or 64 up to a latent of 256)", rows);
  const int mt = rows / 16;
  const size_t smem = latent_mma_smem(D, mt);
  IB_CHECK_ARG(smem <= 220 * 1024, "latent_attention_mma: %d rows of %d values need %zu bytes of shared memory", rows, D, smem);
  const int hpc = heads < rows ? heads : rows;
  dim3 grid((heads + hpc - 1) / hpc, n_units, n_slices);
  auto go = [&](auto kernel) {
    if (smem > 40 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ib::launch(kernel, grid, kWarps * 32, smem, stream, q, *kv, positions, seg_of_token, (const int2*)units, scale, (__nv_bfloat16*)out, part_o, part_ml, heads, rank, D,
               n_slices, slice_keys, status, window);
  };
  auto pick = [&](auto nch) {
    constexpr int NCH = decltype(nch)::value;
    if (mt == 1) go(latent_attention_mma_kernel<NCH, 1>);
    else if (mt == 2) go(latent_attention_mma_kernel<NCH, 2>);
    else if constexpr (NCH <= 2) go(latent_attention_mma_kernel<NCH, 4>);
  };
  if (rank <= 128) pick(std::integral_constant<int, 1>());
  else if (rank <= 256) pick(std::integral_constant<int, 2>());
  else pick(std::integral_constant<int, 4>());
  IB_CHECK_LAUNCH("latent_attention_mma");
  if (n_slices > 1) return ib_latent_combine(part_o, part_ml, out, IB_BF16, T * heads, rank, n_slices, stream);
  return 0;
}
