// Device-side weight layout ("row-chunk tiles") and the accessors every kernel uses.
//
// Host callers hand over GGUF bytes: rows of ceil(K/bs) blocks, each block a
// small struct whose size (18, 34, 144, 210, 136 bytes) is not a multiple of
// 16.  HBM -> shared-memory bulk copies and 128-bit shared loads both want
// 16-byte alignment, so at upload the same bytes are re-ordered (no byte is
// added, dropped or changed) into tiles:
//
//   tile  = 8 consecutive rows x up to QK_TILE_ELEMS consecutive columns
//   chunk = the tiles of one 8-row group, k-tile after k-tile
//   inside a tile the blocks follow one another (block-major), and inside a
//   block the fields of its 8 rows are split into planes, each plane cut into
//   granules of g bytes with the same granule of all 8 rows side by side:
//   [nbt blocks][planes][width/g granules][8 rows][g bytes]
//
//     Q4_0   nibbles 16 B (g 16)          | d 2 B (g 2)                  8 x 18  = 144 B per block
//     Q8_0   int8s   32 B (g 16)          | d 2 B (g 2)                  8 x 34  = 272 B
//     Q4_K   d,dmin,scales 16 B (g 16)    | nibbles 128 B (g 32)         8 x 144 = 1152 B
//     Q6_K   ql+qh  192 B (g 16) | scales 16 B (g 16) | d 2 B (g 2)      8 x 210 = 1680 B
//     IQ4_XS nibbles 128 B (g 16)         | d,scales_h,scales_l 8 B (g 8) 8 x 136 = 1088 B
//     Q5_K   d,dmin,scales 16 B (g 16) | qh 32 B (g 32) | nibbles 128 B (g 32)  8 x 176 = 1408 B
//     Q2_K   scales 16 B (g 16) | qs 64 B (g 16) | d,dmin 4 B (g 4)             8 x 84 = 672 B
//     Q3_K   hmask 32 B (g 16) | qs 64 B (g 16) | scales 12 B (g 4) | d 2 B (g 2)  8 x 110 = 880 B
//     Q8_K   d 4 B (g 4) | qs 256 B (g 16) | bsums 32 B (g 16)                  8 x 292 = 2336 B
//
//   The same 16- or 32-byte group of all 8 rows lies in one 128- or 256-byte
//   span: eight lanes that hold the eight rows read it from HBM as full sectors
//   and from shared memory without bank conflicts, and it is one tensor-core
//   fragment row per lane group.  The 8 x bb bytes of one block column are one
//   contiguous span.  (The accessors below also understand row-major planes,
//   [8 rows][nbt blocks][width], which no format uses any more.)
//
// Every block and every plane of it starts on a 16-byte boundary for any K and
// any row count (8 * width is a multiple of 16 for all widths above), and one
// tile is one contiguous span of HBM, so a single bulk copy stages it.
// Rows are padded up to a multiple of 8 with all-zero blocks (scale 0: they
// contribute exactly 0 and are never written out).
#pragma once
#include <cstdint>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#define QK_TILE_ROWS 8u
#define QK_TILE_ELEMS 4096u

#define QK_T_Q4_0 2
#define QK_T_Q8_0 8
#define QK_T_Q4_K 12
#define QK_T_Q6_K 14
#define QK_T_IQ4_XS 23
#define QK_T_Q5_K 13
#define QK_T_Q2_K 10
#define QK_T_Q3_K 11
#define QK_T_Q8_K 15

struct QkLayout {
  int type;
  uint32_t bs, bb;       // block size (weights) and bytes
  uint32_t nb;           // blocks per row = ceil(cols / bs)
  uint32_t nbt;          // blocks per full k-tile
  uint32_t ktiles;       // k-tiles per chunk
  uint32_t nplanes;
  uint32_t pw[4];        // plane widths, bytes per block
  uint32_t po[4];        // offset of the plane's field inside the GGUF block
  uint32_t pg[4];        // 0: row-major plane; g > 0: interleaved with granule g bytes
  uint32_t bm;           // 1: block-major tile (every plane interleaved, planes of a block adjacent)
  uint32_t rows, cols;   // logical shape of this shard
  uint32_t chunks;       // ceil(rows / 8)
  uint64_t chunk_bytes;  // 8 * nb * bb
  uint64_t tile_bytes;   // 8 * nbt * bb (a full tile)
  uint64_t total_bytes;  // chunks * chunk_bytes
};

static inline bool qk_make_layout(int type, uint64_t rows, uint64_t cols, QkLayout *L) {
  QkLayout l = {};
  l.type = type;
  switch (type) {
    case QK_T_Q4_0:
      l.bs = 32; l.bb = 18; l.nplanes = 2;
      l.pw[0] = 16; l.po[0] = 2; l.pg[0] = 16; l.pw[1] = 2; l.po[1] = 0; l.pg[1] = 2;
      l.bm = 1;
      break;
    case QK_T_Q8_0:
      l.bs = 32; l.bb = 34; l.nplanes = 2;
      l.pw[0] = 32; l.po[0] = 2; l.pg[0] = 16; l.pw[1] = 2; l.po[1] = 0; l.pg[1] = 2;
      l.bm = 1;
      break;
    case QK_T_Q4_K:
      l.bs = 256; l.bb = 144; l.nplanes = 2;
      l.pw[0] = 16; l.po[0] = 0; l.pg[0] = 16; l.pw[1] = 128; l.po[1] = 16; l.pg[1] = 32;
      l.bm = 1;
      break;
    case QK_T_Q5_K:  // d, dmin, scales 16 B | qh 32 B | qs 128 B
      l.bs = 256; l.bb = 176; l.nplanes = 3;
      l.pw[0] = 16; l.po[0] = 0; l.pg[0] = 16; l.pw[1] = 32; l.po[1] = 16; l.pg[1] = 32;
      l.pw[2] = 128; l.po[2] = 48; l.pg[2] = 32;
      l.bm = 1;
      break;
    case QK_T_Q2_K:  // scales 16 B | qs 64 B | d, dmin 4 B
      l.bs = 256; l.bb = 84; l.nplanes = 3;
      l.pw[0] = 16; l.po[0] = 0; l.pg[0] = 16; l.pw[1] = 64; l.po[1] = 16; l.pg[1] = 16;
      l.pw[2] = 4; l.po[2] = 80; l.pg[2] = 4;
      l.bm = 1;
      break;
    case QK_T_Q3_K:  // hmask 32 B | qs 64 B | scales 12 B | d 2 B
      l.bs = 256; l.bb = 110; l.nplanes = 4;
      l.pw[0] = 32; l.po[0] = 0; l.pg[0] = 16; l.pw[1] = 64; l.po[1] = 32; l.pg[1] = 16;
      l.pw[2] = 12; l.po[2] = 96; l.pg[2] = 4; l.pw[3] = 2; l.po[3] = 108; l.pg[3] = 2;
      l.bm = 1;
      break;
    case QK_T_Q8_K:  // d (f32) 4 B | qs 256 B | bsums 32 B
      l.bs = 256; l.bb = 292; l.nplanes = 3;
      l.pw[0] = 4; l.po[0] = 0; l.pg[0] = 4; l.pw[1] = 256; l.po[1] = 4; l.pg[1] = 16;
      l.pw[2] = 32; l.po[2] = 260; l.pg[2] = 16;
      l.bm = 1;
      break;
    case QK_T_Q6_K:
      l.bs = 256; l.bb = 210; l.nplanes = 3;
      l.pw[0] = 192; l.po[0] = 0; l.pg[0] = 16; l.pw[1] = 16; l.po[1] = 192; l.pg[1] = 16;
      l.pw[2] = 2; l.po[2] = 208; l.pg[2] = 2;
      l.bm = 1;
      break;
    case QK_T_IQ4_XS:
      l.bs = 256; l.bb = 136; l.nplanes = 2;
      l.pw[0] = 128; l.po[0] = 8; l.pg[0] = 16; l.pw[1] = 8; l.po[1] = 0; l.pg[1] = 8;
      l.bm = 1;
      break;
    default:
      return false;
  }
  l.rows = (uint32_t)rows;
  l.cols = (uint32_t)cols;
  l.nb = (uint32_t)((cols + l.bs - 1) / l.bs);
  l.nbt = QK_TILE_ELEMS / l.bs;
  l.ktiles = (l.nb + l.nbt - 1) / l.nbt;
  l.chunks = (uint32_t)((rows + QK_TILE_ROWS - 1) / QK_TILE_ROWS);
  l.chunk_bytes = (uint64_t)QK_TILE_ROWS * l.nb * l.bb;
  l.tile_bytes = (uint64_t)QK_TILE_ROWS * l.nbt * l.bb;
  l.total_bytes = l.chunk_bytes * l.chunks;
  *L = l;
  return true;
}

// Blocks held by k-tile `kt` (the last one of a chunk may be short).
__host__ __device__ static inline uint32_t qk_tile_nb(const QkLayout &L, uint32_t kt) {
  uint32_t left = L.nb - kt * L.nbt;
  return left < L.nbt ? left : L.nbt;
}

// Byte offset of tile (chunk, kt) from the start of the buffer.
__host__ __device__ static inline uint64_t qk_tile_offset(const QkLayout &L, uint32_t chunk,
                                                          uint32_t kt) {
  return (uint64_t)chunk * L.chunk_bytes + (uint64_t)kt * L.tile_bytes;
}

// Byte offset of plane p inside a tile holding nbt_this blocks per row.
__host__ __device__ static inline uint32_t qk_plane_offset(const QkLayout &L, uint32_t nbt_this,
                                                           int p) {
  uint32_t w = 0;
  for (int i = 0; i < p; i++) w += L.pw[i];
  return QK_TILE_ROWS * nbt_this * w;
}

// Offset of byte `o` of field-plane p of block (row, blk).  Bytes of one granule
// (the whole field, for a row-major plane) are contiguous.
__host__ __device__ static inline uint64_t qk_byte_offset(const QkLayout &L, uint32_t row,
                                                          uint32_t blk, int p, uint32_t o) {
  uint32_t chunk = row / QK_TILE_ROWS, r = row % QK_TILE_ROWS;
  uint32_t kt = blk / L.nbt, b = blk % L.nbt;
  uint32_t nbt_this = qk_tile_nb(L, kt);
  uint32_t g = L.pg[p];
  if (L.bm) {  // [block][plane][granule][row][g bytes]
    uint32_t before = 0;
    for (int i = 0; i < p; i++) before += L.pw[i];
    return qk_tile_offset(L, chunk, kt) + (uint64_t)b * QK_TILE_ROWS * L.bb +
           (uint64_t)QK_TILE_ROWS * before + (uint64_t)(o / g) * QK_TILE_ROWS * g + (uint64_t)r * g +
           (o % g);
  }
  uint64_t base = qk_tile_offset(L, chunk, kt) + qk_plane_offset(L, nbt_this, p);
  if (g == 0) return base + (uint64_t)(r * nbt_this + b) * L.pw[p] + o;
  return base + (uint64_t)b * QK_TILE_ROWS * L.pw[p] + (uint64_t)(o / g) * QK_TILE_ROWS * g +
         (uint64_t)r * g + (o % g);
}
