// Constants and launcher prototypes shared by the kernel and the host translation units.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace fkb {

struct LaunchParams;

constexpr uint32_t kStagedThreads = 256;
constexpr uint32_t kStagedWarps = kStagedThreads / 32;
constexpr uint32_t kStagedCtasPerSm = 2;
// Shared memory of one warp of a staged CTA: a 288-byte header (eight mbarriers, the plane record), a region for the
// staged source rows — two to four stages of two rows each for RESIZE items, as many as the item's footprint lets fit;
// four stages of one row for POINT items — and two output rows.  14.1 KB per warp, 113 KB per CTA: two CTAs (and the
// kilobyte the system keeps per CTA) fill the 228 KB of an SM.
constexpr uint32_t kSliceHeader = 288;
constexpr uint32_t kMaxTileW = 256;      // widest column segment of an item, in output pixels
constexpr uint32_t kInRowBytes = 1600;   // longest staged source row segment (512 uchar3 pixels + alignment slack)
constexpr uint32_t kInRegionBytes = 7936;
constexpr uint32_t kPointTileU8 = 512;   // pixels per segment of a uchar3 -> uchar3 item
constexpr uint32_t kOutRowBytes = kMaxTileW * 12;  // one output row segment (float3 pixels, or uchar3 with room to spare)
// A planar float row is three segments (one per channel), each followed by 16 spare bytes; a packed row is
// followed by 16 spare bytes.  The spare bytes take the stores of columns that do not exist.
constexpr uint32_t kPlanarSegBytes = kMaxTileW * 4 + 16;
constexpr uint32_t kOutSlotBytes = 3 * kPlanarSegBytes;
constexpr uint32_t kSliceBytes = kSliceHeader + kInRegionBytes + 2 * kOutSlotBytes;
constexpr uint32_t kStagedSmemBytes = kStagedWarps * kSliceBytes;
static_assert(4 * kInRowBytes <= kInRegionBytes, "POINT items stage four rows");
static_assert(kStagedCtasPerSm * (kStagedSmemBytes + 1024) <= 233472, "two CTAs per SM");
constexpr uint32_t kMaxRowsPerItem = 32;
// lut_kernel: a CTA-wide table of 256 rows, 256 bytes apart, each holding 32 copies of one 32-bit word
// {T0[i], T1[i], T2[i], 0} (copy l belongs to lane l and sits in bank l, so a table read never has a bank conflict).  The
// table sits at the absolute shared-memory address 65536, so that the address of a read — 0x10000 | value << 8 | lane << 2
// — is a single byte permute with no addition behind it.  Around it one slice per warp: four mbarriers and a ring of four
// row segments of 512 uchar3 pixels that are transformed in place; as many slices as fit lie below the table, the rest
// above it.  24 warps, one CTA per SM.
constexpr uint32_t kLutThreads = 768;
constexpr uint32_t kLutWarps = kLutThreads / 32;
constexpr uint32_t kLutCtasPerSm = 1;
constexpr uint32_t kLutTableAddr = 65536;  // absolute shared-memory address of the table
constexpr uint32_t kLutBytes = 256 * 256;  // 256 values, rows 256 bytes apart (32 lane copies of a 4-byte entry, then unused)
constexpr uint32_t kLutSegBytes = 1536;
constexpr uint32_t kLutStages = 4;
constexpr uint32_t kLutSliceBytes = 64 + kLutStages * kLutSegBytes;
// dynamic shared memory: enough for the slices above the table when only nine fit below it (the dynamic region starts
// after the kernel's static variables and whatever the system reserves; the kernel checks the layout it finds)
constexpr uint32_t kLutSmemBytes = kLutTableAddr + kLutBytes + (kLutWarps - 9) * kLutSliceBytes;

constexpr uint64_t kTinyLaunchPixels = 100000;  // launches below this many output pixels take the general kernel
constexpr uint64_t kPdlMinPixels = 200000;      // launches of at least this many output pixels allow programmatic stream serialisation
constexpr uint64_t kJoinGeneralPixels = 400000; // pipelined planes below this many pixels join a general kernel that runs anyway

cudaError_t launch_staged(const LaunchParams& p, uint32_t grid, cudaStream_t stream);
cudaError_t launch_lut(const LaunchParams& p, uint32_t grid, cudaStream_t stream);
cudaError_t launch_nv12(const LaunchParams& p, dim3 grid, cudaStream_t stream);
cudaError_t launch_gather(const LaunchParams& p, dim3 grid, int pixels_per_thread, cudaStream_t stream);
cudaError_t launch_gather4(const LaunchParams& p, dim3 grid, cudaStream_t stream);
cudaError_t status_word_address(int** out);

}  // namespace fkb
