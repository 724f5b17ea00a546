// Host helpers that build TMA tensor maps for [batch, head, sequence, channel] tensors.
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace kfa {

// True when a 16-bit tensor with these element strides (order: batch, head, sequence,
// channel) can be addressed by a tiled tensor map: channel-contiguous, 16-byte aligned
// base, and every other stride a positive multiple of 16 bytes.
bool tma_compatible(const void* ptr, const int64_t* strides, int64_t B, int64_t H, int64_t S);

// Encodes a rank-4 map with dimensions (channel, sequence, head, batch), a box of
// `box_channels` x `box_rows` x 1 x 1 and the 128-byte shared-memory swizzle.
// Out-of-range elements read as zero.  Returns false when the driver rejects it.
bool encode_bhsd_map(CUtensorMap* map, const void* ptr, CUtensorMapDataType dtype, int64_t D, int64_t S, int64_t H,
                     int64_t B, const int64_t* strides, int box_channels, int box_rows);

}  // namespace kfa
