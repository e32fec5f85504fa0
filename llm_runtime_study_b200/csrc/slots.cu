// The per-request slot records on the device.
//
// A request that is being decoded owns one record of kSlotWords 32-bit words in a table of
// max_requests + 1 records (the last one belongs to nobody: rows that pad a batch up to the size
// of its captured graph point there).  The reference keeps the same things on the host, per
// request: the number of tokens in the cache (mini_llm/cache/lengths.py:8-43), the token sampled
// last and the index of the next one (mini_llm/generation.py:56-70), a random generator
// (mini_llm/sampling.py:94-101).  Held on the device they let a decode step start from nothing but
// the list of slots in the batch: the step's token ids, positions and lengths are read out of the
// records here, and the sampling kernels (sampling.cu) write the chosen token back.
//
//   word 0  position     tokens of the request in the cache = position of its next token
//   word 1  last token   sampled by the step before, not in the cache yet
//   word 2  temperature  (float bits)     word 3  top_k (0: off)      word 4  top_p (float bits)
//   word 5  seed, low    word 6  seed, high                           word 7  counter: index of the next token to draw
//   word 8  live         1 while a request holds the slot, 0 for the padding record
#include "common.cuh"
#include "slots.h"

namespace b200 {

// records[slots[i]] = staged[i] for i < n: how the host writes the records of the requests in a
// step that it has packed itself (prompt portions), in the same upload as the step's other metadata.
__global__ void slot_store_kernel(int* __restrict__ records, const int* __restrict__ staged,
                                  const int* __restrict__ slots, int n) {
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n * kSlotWords) return;
  const int row = i / kSlotWords, word = i - row * kSlotWords;
  records[static_cast<size_t>(slots[row]) * kSlotWords + word] = staged[i];
}

// For every row of a batch of single decoded tokens: the token to feed, its position, and the
// request's length after this step, taken from the row's record; the record's position advances.
// A record that is not live (padding) gives token 0 at position 0 of a sequence of length 0, which
// the cache write and the attention kernels skip.
__global__ void slot_load_kernel(int* __restrict__ records, const int* __restrict__ slots, int* __restrict__ token_ids,
                                 int* __restrict__ positions, int* __restrict__ kv_len, int n) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= n) return;
  int* rec = records + static_cast<size_t>(slots[row]) * kSlotWords;
  const bool live = rec[kSlotLive] != 0;
  const int pos = live ? rec[kSlotPosition] : 0;
  const int token = live ? rec[kSlotLastToken] : 0;
  token_ids[row] = token < 0 ? 0 : token;   // a refused draw (-1: non-finite logits) is reported by the host; never index with it
  positions[row] = pos;
  kv_len[row] = live ? pos + 1 : 0;
  if (live) rec[kSlotPosition] = pos + 1;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_slot_words() { return kSlotWords; }

extern "C" int b200_slot_store(int* records, const int* staged, const int* slots, int n, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int threads = 128, total = n * kSlotWords;
  launch(slot_store_kernel, dim3((total + threads - 1) / threads), dim3(threads), 0, stream, records, staged, slots, n);
  return launch_status();
}

extern "C" int b200_slot_load(int* records, const int* slots, int* token_ids, int* positions, int* kv_len, int n,
                              cudaStream_t stream) {
  if (n <= 0) return 0;
  const int threads = 64;
  launch(slot_load_kernel, dim3((n + threads - 1) / threads), dim3(threads), 0, stream, records, slots, token_ids, positions,
         kv_len, n);
  return launch_status();
}
