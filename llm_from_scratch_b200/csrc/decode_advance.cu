// Device-side step of the decode metadata, so that several decode steps can run back to back without the
// host in between (the host side of one step is ModelRunner.prepare_decode, engine/model_runner.py:253-278:
// input id = last sampled token, context length = tokens so far, slot = position of the new token in the
// sequence's last block).  After a step sampled `sampled[i]` for row i, the next step's inputs are
//   input_ids[i]    = sampled[i]
//   context_lens[i] = context_lens[i] + 1
//   slot_mapping[i] = block_tables[i, (len - 1) / block_size] * block_size + (len - 1) % block_size
// where the block table already holds every block the coming steps write into (the host opens them
// before the first step).  The sampled tokens are also appended to a history row for the host.
#include "common.cuh"

namespace b200 {
namespace {

__global__ void decode_advance_kernel(const int64_t* __restrict__ sampled, int64_t* __restrict__ input_ids,
                                      int64_t* __restrict__ context_lens, int64_t* __restrict__ slot_mapping,
                                      const int32_t* __restrict__ block_tables, int64_t bt_stride, int block_size,
                                      int64_t num_blocks, int n, int64_t* __restrict__ history, int32_t* status) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t tok = sampled[i];
  if (history) history[i] = tok;
  input_ids[i] = tok;
  const int64_t len = context_lens[i] + 1;
  const int64_t blk = (len - 1) / block_size;
  int64_t slot = -1;
  if (blk < bt_stride) {
    const int64_t id = block_tables[static_cast<int64_t>(i) * bt_stride + blk];
    if (id >= 0 && id < num_blocks)
      slot = id * block_size + (len - 1) % block_size;
    else
      report(status, B200_ERR_BOUNDS);
  } else {
    report(status, B200_ERR_BOUNDS);     // the host asked for more steps than the table has room for
  }
  context_lens[i] = len;
  slot_mapping[i] = slot;
}

}  // namespace
}  // namespace b200

extern "C" int b200_decode_advance(const int64_t* sampled, int64_t* input_ids, int64_t* context_lens,
                                   int64_t* slot_mapping, const int32_t* block_tables, int64_t bt_stride,
                                   int32_t block_size, int64_t num_blocks, int32_t num_seqs, int64_t* history,
                                   int32_t* status, void* stream) {
  using namespace b200;
  if (num_seqs < 0 || block_size <= 0 || bt_stride <= 0 || num_blocks <= 0) return B200_ERR_ARG;
  if (num_seqs == 0) return B200_OK;
  if (!sampled || !input_ids || !context_lens || !slot_mapping || !block_tables) return B200_ERR_ARG;
  decode_advance_kernel<<<(num_seqs + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      sampled, input_ids, context_lens, slot_mapping, block_tables, bt_stride, block_size, num_blocks, num_seqs,
      history, status);
  return launch_result();
}

// ---------------------------------------------------------------------------------------------
// Device-resident block tables: instead of uploading the whole [batch, max_blocks] table every decode
// step (ModelRunner.prepare_decode rebuilds and ships it, engine/model_runner.py:263-268), the host sends
// only the entries that changed since the previous step — normally one new block per sequence every
// block_size steps — as (row, column, block id) triples that this kernel writes into the table.
namespace b200 {
namespace {

__global__ void block_table_patch_kernel(const int32_t* __restrict__ patches, int count,
                                         int32_t* __restrict__ tables, int64_t bt_stride, int rows,
                                         int32_t* status) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= count) return;
  const int row = patches[3 * p], col = patches[3 * p + 1], val = patches[3 * p + 2];
  if (row < 0 || row >= rows || col < 0 || col >= bt_stride) {
    report(status, B200_ERR_BOUNDS);
    return;
  }
  tables[static_cast<int64_t>(row) * bt_stride + col] = val;
}

}  // namespace
}  // namespace b200

extern "C" int b200_block_table_patch(const int32_t* patches, int32_t count, int32_t* block_tables,
                                      int64_t bt_stride, int32_t rows, int32_t* status, void* stream) {
  using namespace b200;
  if (count < 0 || bt_stride <= 0 || rows < 0) return B200_ERR_ARG;
  if (count == 0) return B200_OK;
  if (!patches || !block_tables) return B200_ERR_ARG;
  block_table_patch_kernel<<<(count + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      patches, count, block_tables, bt_stride, rows, status);
  return launch_result();
}
