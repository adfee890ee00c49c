// How kernels address one layer's keys and values inside a paged pool.
//
// A pool is [entries][num_pages][2 (K, V)][kv_heads][page_size][head_dim] (one layer's pages lie together);
// a view fixes the entry (the layer), so
//   K(page, head, slot, d) = base + page * page_stride + (head * page_size + slot) * head_dim + d
//   V(...)                 = the same + v_offset
// The page of position p of segment s is block_table[s * table_stride + p / page_size].
// The reference uses the same block-major idea with a fixed page of 16
// (crates/kir/src/cuda/attention/prim.rs:217; docs/specrt-scheduler.md:20-22).
#pragma once
#include "common.cuh"

struct IbKvView {
  void* base;              // first element of this layer's K in page 0
  long long page_stride;   // elements between consecutive pages
  long long v_offset;      // elements from a K element to the V element of the same place
  const int* block_table;  // [segments][table_stride]
  int table_stride;
  int page_size;
  int num_pages;
  int kv_heads;
  int head_dim;
  int dtype;  // IB_F32 or IB_BF16
};

// What the tensor-core attention kernels do to a head's finished sum, beyond the plain softmax: the score of the sink (an extra term of
// the denominator without a value) per head, a gate per (token, head) and a constant on the output, and the output's row length when
// the heads are the first columns of a wider buffer. All zero: a sink of score 0, no gate, factor 1, rows of heads * head_dim.
struct IbAttnTail {
  const float* sink_values;  // float32 [heads], in natural units (not scaled), or null
  const float* gate;         // float32 partial sums [gate_parts][tokens][gate_row], offset to the first head's column, or null:
  int gate_parts;            //   head h's output is multiplied by sigmoid(sum over the parts of gate[t][h])
  int gate_row;
  long long gate_stride;     // elements between consecutive parts
  float out_scale;           // 0 stands for 1
  int out_row;               // elements per output row; 0 stands for heads * head_dim
};

namespace ib {

// The first position that `pos` sees. window > 0: itself and the window - 1 before it; window < 0: the earlier positions of its own
// block of -window positions, blocks counted from position 0; 0: every earlier position.
__device__ __forceinline__ int first_visible(int pos, int window) {
  return window > 0 ? max(0, pos - window + 1) : window < 0 ? pos - pos % (-window) : 0;
}

// The factor on head h's output for token t: out_scale * sigmoid(gate).
__device__ __forceinline__ float tail_factor(const IbAttnTail& tail, int t, int h) {
  float f = tail.out_scale != 0.f ? tail.out_scale : 1.f;
  if (tail.gate) {
    const float* g = tail.gate + (size_t)t * tail.gate_row + h;
    float z = g[0];
    for (int p = 1; p < tail.gate_parts; p++) z += g[(size_t)p * tail.gate_stride];
    f *= 1.f / (1.f + __expf(-z));
  }
  return f;
}

// Element offset of (position, kv head) in a view, or -1 when the table has no valid page there.
__device__ __forceinline__ long long kv_offset(const IbKvView& kv, int seg, int pos, int head) {
  int page = kv.block_table[(size_t)seg * kv.table_stride + pos / kv.page_size];
  if (page < 0 || page >= kv.num_pages) return -1;
  return (long long)page * kv.page_stride + ((long long)head * kv.page_size + pos % kv.page_size) * kv.head_dim;
}

}  // namespace ib
