// TMA tensor maps of bfloat16 tensors, made once per (address, shape, box) and cached.
#pragma once

#include <cuda.h>

// A bfloat16 tensor of `rank` (2 or 3) dimensions, innermost first: extents `dims`, byte strides of
// dimensions 1.. in `strides` (multiples of 16), boxes of `box` elements; with the 128-byte swizzle
// when `swizzle128` (the innermost box extent is then 64 elements), else unswizzled. Elements outside
// the tensor read as zero and are not written. Returns 0, or 1 with the message in ti_last_error().
int ti_tensor_map_bf16(CUtensorMap* out, const void* ptr, int rank, const unsigned long long* dims,
                       const unsigned long long* strides, const unsigned* box, bool swizzle128);
