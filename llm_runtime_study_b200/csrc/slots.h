// Layout of a per-request slot record (32-bit words); see slots.cu.  The six words from
// kSlotSampling on are, in this order, what the sampling kernels take per row of logits.
#pragma once

namespace b200 {

constexpr int kSlotWords = 12;        // a record is 48 bytes: a multiple of 16
constexpr int kSlotPosition = 0;
constexpr int kSlotLastToken = 1;
constexpr int kSlotSampling = 2;      // temperature bits, top_k, top_p bits, seed low, seed high, counter
constexpr int kSlotCounter = 7;
constexpr int kSlotLive = 8;

}  // namespace b200
