// Internal: GPU-side gather of crop rows from pinned host memory (see host_gather.cu).
#pragma once
#include <cstdint>

namespace tlb {

struct GatherItem {
    unsigned long long src;  // device-visible address of the crop's first byte (row 0, column x)
    unsigned long long dst_off;  // byte offset of the packed crop in the destination buffer (16-byte aligned)
    unsigned src_pitch;      // bytes between source rows (image width * 3)
    unsigned row_bytes;      // crop width * 3
    unsigned rows;           // crop height
    unsigned dst_pitch;      // bytes between packed rows (multiple of 48: a whole number of pixels and of 16)
};

// Returns a cudaError_t as int.  grid = n x ceil(max_rows / 16).
int launch_gather(const GatherItem* items_dev, int n, unsigned max_rows, unsigned char* dst, void* stream);

}  // namespace tlb
