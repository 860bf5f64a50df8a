// Host-side pieces of the decode attention shared with the fused layer path: the plan of a call, its workspace
// layout, and the three launches (query absorption, cache stream, merge) as separate functions.
#pragma once

#include "common.cuh"
#include "fused.cuh"

namespace lsvd {

struct HeadPlan {
  int32_t k_col, v_col;      // byte offsets of the head inside a K / V cache row
  int16_t nk, nv;            // 16-entry chunks of K and V
  int16_t chunk_tiles;       // tiles per work item of this head
  int16_t parts;             // work items per request (bounded with max_len_in_batch)
  int32_t part_off;          // first item of this head inside a request's item list
  int32_t acc_off;           // float offset of this head's partial accumulators inside a request's block
};

struct HostPlan {
  HeadPlan head[LSVD_MAX_HEADS];
  int item_bytes = 0;
  int items_per_request = 0, acc_per_request = 0;
  int64_t total_items = 0;
  int num_blocks = 0;
};

struct WorkspaceLayout {
  size_t qlimb, qstep, queue, san, part_ml, part_acc, total;
};

struct AttnLaunch {
  HostPlan hp;
  WorkspaceLayout wl;
};

int attn_prepare(const lsvd_attn_decode_args* a, AttnLaunch* L);
float attn_score_scale(const lsvd_attn_decode_args* a);
int attn_launch_absorb(const lsvd_attn_decode_args* a, const AttnLaunch& L, cudaStream_t st);
int attn_launch_stream(const lsvd_attn_decode_args* a, const AttnLaunch& L, cudaStream_t st);
int attn_launch_merge(const lsvd_attn_decode_args* a, const AttnLaunch& L, cudaStream_t st);
void attn_fill_merge(const lsvd_attn_decode_args* a, const AttnLaunch& L, FMerge* mg);
void attn_workspace_views(const lsvd_attn_decode_args* a, const AttnLaunch& L, uint4** qlimb, float** qstep, int32_t** queue);

}  // namespace lsvd
