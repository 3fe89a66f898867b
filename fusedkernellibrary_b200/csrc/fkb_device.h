/* Device-resident form of a plan: what fkb_plan_create uploads and the kernels read.
 *
 * The reference keeps the per-plane parameters in a compile-time-sized array inside the
 * kernel arguments (operation_model/batch_operations.h:98-102, executor_kernels.h:25-29),
 * which caps a launch at the 32 KB argument space.  Here they are rows of a table in
 * global memory, read once per thread block, so the batch size is a run-time value.
 */
#ifndef FKB_DEVICE_H
#define FKB_DEVICE_H

#include <math.h>
#include <stdint.h>

namespace fkb {

constexpr uint32_t CHAIN_INTERPRET = 0xFFFFFFFFu; /* see the end of this file */
/* Flag on a compiled chain of at most seven operations: every arithmetic operation has the same parameter for the three
   channels (Mul by 1.4, Sub 0.5, Div by 255: the common case), so that the kernel fetches one parameter pair per operation
   instead of three. */
constexpr uint32_t CHAIN_UNIFORM = 0x80000000u;

/* How a plane is processed (chosen on the host from formats, sizes and alignment). */
enum PlaneClass : uint32_t {
    CLASS_GENERIC = 0,       /* one thread per output pixel, scalar accesses; always valid   */
    CLASS_FLAT_U8_F32 = 1,   /* no geometry stage, 4 whole pixels per thread, vector accesses */
    CLASS_FLAT_F32_F32 = 2,
    CLASS_FLAT_U8_U8 = 3,
    CLASS_RESIZE_U8_PLANAR = 4, /* bilinear, 4 adjacent output pixels per thread             */
    CLASS_RESIZE_U8_PACKED = 5,
    CLASS_RESIZE_NV12_PACKED = 6,
    CLASS_RESIZE_U8_PLANAR_STAGED = 7, /* bilinear from a source footprint staged in shared memory */
    CLASS_RESIZE_U8_PACKED_STAGED = 8,
    CLASS_RESIZE_NV12_PACKED_STAGED = 9, /* NV12 taps from luma and chroma rows staged in shared memory */
    CLASS_COUNT = 10,
    CLASS_MIXED = 0xFF       /* launch-level only: planes of several classes in one grid     */
};

struct alignas(16) DevPlane {
    const uint8_t* src;      /* image base (not offset by the crop)                           */
    uint8_t* dst;
    uint32_t src_pitch;
    uint32_t src_height;     /* NV12: chroma plane begins at src + src_pitch * src_height     */
    int32_t crop_x, crop_y, crop_w, crop_h;
    uint32_t dst_w, dst_h, dst_pitch, dst_cstride;
    float fx, fy;            /* resize.h:108-112: source step per output element              */
    int32_t x1, y1, x2, y2;  /* region of interest, inclusive (resize.h:150-158); the whole   */
                             /* output for IGNORE_AR                                          */
    uint32_t seq;
    uint32_t plane_class;
    uint32_t seg_pixels;     /* FLAT classes: pixels per contiguous segment; staged NV12:     */
                             /* output rows per work item (band); staged uchar3: index, within */
                             /* the whole region of interest, of this column tile's first     */
                             /* region column (a region wider than a block's columns is cut   */
                             /* into tiles, each a DevPlane of its own over the same source)  */
    uint32_t n_segs;         /* FLAT classes: 1 (dense plane) or dst_h (one segment per row); */
                             /* staged uchar3 resize: 1 when the last band also fills the     */
                             /* rows outside the region (no store-only items)                 */
    /* RESIZE classes: tiling of the region of interest (see ResizeTiling) */
    uint32_t roi_items;      /* work items that interpolate; the rest fill background rows    */
    uint32_t tiles_x;        /* STAGED classes: output rows per work item (band)               */
    uint32_t gw;             /* CLASS_GENERIC: the source image's width (border handling)      */
    uint32_t rs;
};
static_assert(sizeof(DevPlane) == 112, "DevPlane layout");

struct alignas(16) DevOp {
    int32_t opcode;
    float p[3];
};
static_assert(sizeof(DevOp) == 16, "DevOp layout");

struct alignas(16) DevSeq {
    int32_t src_format, dst_format, resize_mode;
    int32_t n_ops, n_pre, ops_begin; /* ops_begin: index of the first op in the op table      */
    int32_t pre_kind;                /* PRE_* below                                           */
    uint32_t chain;                  /* the continuation as a compiled chain, or CHAIN_INTERPRET */
    float bg[3];
    float one;                       /* 1.0f, read at run time by the packed additions         */
    float bg_out[3];                 /* bg after the operations that follow the geometry stage  */
    uint32_t swap_uv;                /* 1: the chroma pair of a tap is stored V,U (NV21)         */
    /* read-back operations that only the one-pixel-per-thread body takes */
    int32_t border_mode;             /* fkb_border_mode                                          */
    int32_t deinterlace;             /* fkb_deinterlace_mode                                     */
    float border_value[3];
    float transform[9];              /* FKB_GEOMETRY_WARP_*: rows of three                        */
    /* FKB_SRC_P010 / P210 / Y210 / UYVY: the read converts to RGB itself (the conversion is dropped from the
       operation list) */
    int32_t yuv_kind;                /* PRE_YUV_* of that conversion, 0 for the other formats    */
    uint32_t yuv_shift;              /* 6 for the 10-bit layouts, else 0                         */
};
static_assert(sizeof(DevSeq) == 128, "DevSeq layout");

enum PreKind : int32_t {
    PRE_IDENTITY = 0, /* nothing, or only exact uchar->float casts, before interpolation      */
    PRE_YUV_BT709 = 1,/* exactly ConvertYUVToRGB<NV12,Full,bt709,false,float3>                */
    PRE_GENERAL = 2,  /* any other chain: interpreted per tap (generic class only)           */
    PRE_YUV_BT601 = 3,/* exactly ConvertYUVToRGB<PF,Full,bt601,false,float3>                   */
    PRE_YUV_BT2020 = 4/* exactly ConvertYUVToRGB<PF,Full,bt2020,false,float3>                  */
};

/* Rows of `pitch` bytes that a source image of `height` pixel rows occupies, by format. */
__host__ __device__ inline uint32_t source_rows(int src_format, uint32_t height) {
    return (src_format == FKB_SRC_NV12 || src_format == FKB_SRC_NV21 || src_format == FKB_SRC_P010) ? height + (height + 1u) / 2u
           : src_format == FKB_SRC_P210 ? 2u * height : height;
}
/* Bytes of the longest row of any plane of the image. */
__host__ __device__ inline uint64_t source_row_bytes(int src_format, uint32_t width) {
    const uint64_t pairs = ((uint64_t)width + 1u) / 2u;
    switch (src_format) {
        case FKB_SRC_U8X3: return 3ull * width;
        case FKB_SRC_F32X3: return 12ull * width;
        case FKB_SRC_NV12: case FKB_SRC_NV21: return 2ull * pairs;
        case FKB_SRC_P010: case FKB_SRC_P210: return 4ull * pairs;
        case FKB_SRC_Y210: return 8ull * pairs;
        default: return 4ull * pairs; /* FKB_SRC_UYVY */
    }
}

constexpr int INLINE_MAX_OPS = 16;

/* Kernel argument block (passed by value). */
struct LaunchArgs {
    const DevPlane* planes;
    const DevSeq* seqs;
    const DevOp* ops;
    const uint4* items;         /* one entry per thread block: plane, tile within the plane,  */
                                /* sequence | operations << 16, first operation; the staged    */
                                /* uchar3 classes have two per block, the second being the     */
                                /* first byte to copy, rows | row bytes << 16, source pitch    */
    uint32_t n_planes;
    uint32_t wait_limit_us;     /* longest wait of a block for its asynchronous copies (global timer) */
    uint32_t total_items;
    uint32_t max_seq_ops;       /* longest sequence: sizes the shared-memory op cache         */
    uint32_t block_threads;     /* threads per block of this launch (multiple of 32, <= 256)  */
    uint32_t staged_bytes;      /* STAGED classes: shared memory behind the operation cache    */
    uint32_t inline_plane;      /* 1: a plan of one plane whose descriptors travel in the      */
                                /* kernel arguments below; block b is tile b of that plane     */
    uint32_t test_extra_bytes;  /* TEST ONLY: bytes a block expects beyond what its copies deliver   */
    uint32_t prefetch_items;    /* > 0: one dense float3 -> float3 element-wise plane with a long chain; a block asks the L2 */
                                /* for the bytes of the work item this far ahead of its own                                   */
    uint32_t nv12_early;        /* staged NV12 class: 1 when a work item has NV12_ITEM_WORDS table words: the entry, then the     */
                                /* luma and chroma base pointers, pitch / row bytes / spans / luma rows, and one bit per source */
                                /* row of the luma and chroma spans for the rows to copy                                         */
    uint32_t tiled_copies;      /* staged uchar3 classes: 1 when a band's second table entry names a tensor map (index, 0,     */
                                /* bytes of the box, x | y << 16) instead of the rows of per-row copies                       */
    const unsigned char* tmaps; /* the plan's tensor maps, TENSOR_MAP_BYTES each                                             */
    uint32_t test_shrink_bounds;/* TEST ONLY, bounds-checking build: destination rows the checker pretends are missing */
    uint32_t* status;           /* one word in the plan's device block: 0, or a STATUS_* code  */
    DevPlane plane0;            /* inline_plane: the plane, its sequence and its operations    */
    DevSeq seq0;
    DevOp ops0[INLINE_MAX_OPS];
};

constexpr int BLOCK_THREADS = 256;
constexpr int PX_PER_THREAD = 4;
constexpr int FLAT_QUADS_U8 = 4;
/* FLAT classes: runs of four pixels per thread.  A thread has the raw words of all its runs in
 * flight before it computes the first; a uchar3 run is three words, so four runs are cheap to hold,
 * a float3 run is twelve (two runs measured slower than one: 36.9 -> 42.8 us on one 4K float3 Add). */
__host__ __device__ constexpr int flat_quads(bool src_is_u8) { return src_is_u8 ? FLAT_QUADS_U8 : 1; }
/* FLAT classes: pixels per work item */
__host__ __device__ constexpr int flat_item_pixels(bool src_is_u8) { return BLOCK_THREADS * PX_PER_THREAD * flat_quads(src_is_u8); }
constexpr int ITEM_PIXELS_GENERIC = BLOCK_THREADS;
/* FLAT float3 -> float3, one dense plane: from this many arithmetic operations per value a block prefetches the work item
   FLAT_PREFETCH_ITEMS ahead into the L2 (the blocks a B200 holds at five per SM, 9 MB; twice and four times as far measured
   the same or worse).  A 4K image: one operation 34.9 us with and without, four 38.0 -> 34.9, sixteen 38.6 -> 35.1. */
constexpr uint32_t FLAT_PREFETCH_MIN_OPS = 2;
constexpr uint32_t FLAT_PREFETCH_ITEMS = 148u * 5u;

/* Device-only opcode: division by a plan-time constant, lowered from FKB_OP_DIV when the host
 * has proven the three-instruction form exact.  Takes two op slots: {-p}, then {1/p}. */
constexpr int32_t DEV_OP_DIV_BY_CONSTANT = 16;
/* Device-only opcode: the next p[1] slots (1 or 2 of Mul, Sub, Add) run p[0] times; both counts are
 * stored as integer bit patterns. */
constexpr int32_t DEV_OP_REPEAT = 17;

/* RESIZE classes.  Only the region of interest [x1,x2] x [y1,y2] of a plane is interpolated;
 * everything else receives one constant (the default value after the continuation).  Threads
 * are therefore laid over the region of interest alone: a thread owns one group of four
 * adjacent output columns and walks RESIZE_ROWS_PER_THREAD rows `rs` apart, so its horizontal
 * taps and weights are computed once.  A block covers `gw` column groups x (rs *
 * RESIZE_ROWS_PER_THREAD) rows and also fills the background to the left and right of its
 * rows; rows above and below the region are filled by separate, store-only work items of
 * BG_GROUPS_PER_ITEM column groups each. */
constexpr int RESIZE_ROWS_PER_THREAD = 8;
constexpr int RESIZE_PX = 4; /* output columns per thread in the interpolating items */
constexpr int BG_GROUPS_PER_THREAD = 8;

struct ResizeTiling {
    uint32_t g_lo, n_groups; /* first column group touching the region, and how many do        */
    uint32_t n_rows;         /* rows of the region                                             */
    uint32_t gw;             /* threads across a block: each owns RESIZE_PX columns gw apart   */
    uint32_t rs;             /* row slots per block: active threads = gw * rs                  */
    uint32_t tiles_x, tiles_y;
    uint32_t roi_items;      /* tiles_x * tiles_y                                              */
    uint32_t bg_items;       /* store-only items for the rows outside the region               */
};
/* Staged uchar3 resize: the bytes of a crop row that the taps of region columns
 * [col0, col0 + n_cols) touch, widened to 16-byte boundaries (what one bulk copy fetches per
 * source row).  First taps are floor(column * fx) in binary32 (resize.h:183-194,
 * interpolation.h:66-67); host and device evaluate the same expression. */
struct StagedSpan {
    int sx0;            /* first source column staged, relative to the crop            */
    uint32_t row_first; /* byte offset of the copy within a source row                 */
    uint32_t phase;     /* byte of column sx0 within the copy                          */
    uint32_t row_len;   /* bytes per copied row, a multiple of 16                      */
};
#if defined(__CUDACC__)
__host__ __device__
#endif
inline StagedSpan staged_span(int crop_x, int crop_w, uint32_t col0, uint32_t n_cols, float fx) {
    StagedSpan s;
#if defined(__CUDA_ARCH__)
    s.sx0 = __float2int_rd(__fmul_rn((float)col0, fx));
    int sx1 = __float2int_rd(__fmul_rn((float)(col0 + n_cols - 1u), fx)) + 1;
#else
    s.sx0 = (int)floorf((float)col0 * fx);
    int sx1 = (int)floorf((float)(col0 + n_cols - 1u) * fx) + 1;
#endif
    if (sx1 > crop_w - 1) sx1 = crop_w - 1;
    if (sx1 < s.sx0) sx1 = s.sx0;
    const uint32_t b0 = (uint32_t)(crop_x + s.sx0) * 3u;
    s.row_first = b0 & ~15u;
    s.phase = b0 - s.row_first;
    s.row_len = (s.phase + (uint32_t)(sx1 - s.sx0 + 1) * 3u + 15u) & ~15u;
    return s;
}

#if defined(__CUDACC__)
__host__ __device__
#endif
inline ResizeTiling resize_tiling(uint32_t dst_w, uint32_t dst_h, int x1, int y1, int x2, int y2,
                                  uint32_t block_threads) {
    ResizeTiling t;
    const uint64_t per_item = (uint64_t)block_threads * BG_GROUPS_PER_THREAD;
    if (x2 < x1 || y2 < y1) {
        /* An empty region (a PRESERVE_AR target that rounds to zero columns or rows, resize.h:196-221):
           no interpolating items, every row is filled by store-only items. */
        t.g_lo = 0; t.n_groups = 0; t.n_rows = 0; t.gw = block_threads; t.rs = 1; t.tiles_x = 1; t.tiles_y = 0;
        t.roi_items = 0;
        t.bg_items = (uint32_t)(((uint64_t)dst_h * (dst_w / PX_PER_THREAD) + per_item - 1) / per_item);
        return t;
    }
    t.g_lo = (uint32_t)x1 / PX_PER_THREAD;
    t.n_groups = (uint32_t)x2 / PX_PER_THREAD - t.g_lo + 1;
    t.n_rows = (uint32_t)(y2 - y1 + 1);
    const uint32_t col_threads = (t.n_groups * PX_PER_THREAD + RESIZE_PX - 1) / RESIZE_PX;
    t.tiles_x = (col_threads + block_threads - 1) / block_threads;
    t.gw = (col_threads + t.tiles_x - 1) / t.tiles_x;
    t.rs = block_threads / t.gw;
    const uint32_t rows = t.rs * RESIZE_ROWS_PER_THREAD;
    t.tiles_y = (t.n_rows + rows - 1) / rows;
    t.roi_items = t.tiles_x * t.tiles_y;
    const uint64_t bg_groups = (uint64_t)(dst_h - t.n_rows) * (dst_w / PX_PER_THREAD);
    t.bg_items = (uint32_t)((bg_groups + per_item - 1) / per_item);
    return t;
}

/* STAGED classes: a work item is a band of `band_rows` output rows of the region of interest,
 * all columns; its source footprint (whole crop rows, widened to 16-byte boundaries) sits in
 * shared memory behind a 16-byte mbarrier slot and a table of per-row vertical taps. */
constexpr uint32_t STAGED_BAND_PIXELS = 5376; /* output pixels per band, about (4480 / 5376 / 6272 / 7168 / 8960: 152.0 / 152.6 / 153.3 / 154.2 / 156.1 us on the 1024-crop batch) */
constexpr uint32_t STAGED_MIN_BAND_PIXELS = 448; /* bands of a plan with a small grid are halved down to this       */
constexpr uint32_t SMALL_GRID_BLOCKS = 148;      /* fewer blocks than this (one per SM of a B200): shorter bands        */
constexpr uint32_t STAGED_MAX_ROWS = 64;          /* output rows per band                        */
constexpr uint32_t STAGED_MAX_STAGE_BYTES = 40 * 1024u; /* five blocks of it fit one SM */
constexpr uint32_t STAGED_HEADER_BYTES = 16 + STAGED_MAX_ROWS * 32;
/* the staged uchar3 classes round it up to 128 bytes: a tiled bulk copy wants its destination on such a boundary */
constexpr uint32_t STAGED_U8_HEADER_BYTES = (STAGED_HEADER_BYTES + 127u) & ~127u;
/* A band's source rows as ONE tiled bulk copy through a tensor map of its plane (box = row bytes x rows) instead of one
   bulk copy per row: rows of at most 256 eight-byte elements, at most 256 rows, coordinates that fit 16 bits. */
constexpr uint32_t TILED_MAX_ROW_BYTES = 256u * 8u;
constexpr uint32_t TILED_MAX_ROWS = 256u;
constexpr uint32_t TENSOR_MAP_BYTES = 128u;
constexpr uint32_t NV12_MAX_STAGE_BYTES = 50 * 1024u; /* luma and chroma rows of a band tile; four blocks per SM.  The body is bound
                                                         by the latency of its shared-memory taps: two rows in flight per thread at 64 registers and
                                                         four blocks measured 100.4 us on 32 4K frames against 102.5 with one row at 48 registers
                                                         and five blocks (two rows at 48 registers spill: 106.2), and 97.5 with the larger stage
                                                         that four blocks leave room for (three rows 103.2; four rows at three blocks 115.5). */
constexpr uint32_t NV12_ITEM_WORDS = 8;           /* 16-byte table words per work item of a staged NV12 plan (LaunchArgs::nv12_early) */
constexpr uint32_t NV12_MAX_SPAN = 256;           /* source rows between a band's first and last tap */
constexpr uint32_t STAGED_FOLD_BG_GROUPS = 1024;  /* at most this many outside groups: no store-only items */
constexpr uint32_t STATUS_STAGED_WAIT_TIMEOUT = 1; /* a bulk copy did not complete in time        */
/* bounds-checking build only: an access outside what the block's plane allows was refused (the largest code is kept) */
constexpr uint32_t STATUS_BOUNDS_SOURCE = 2, STATUS_BOUNDS_DESTINATION = 3, STATUS_BOUNDS_SHARED = 4;

/* Compile-time operation chains.  A chain is a list of 4-bit operation codes, first operation
 * in the lowest nibble, 0 terminates.  Kernels are instantiated for the chains in
 * FKB_CHAIN_MENU; any other sequence runs through the interpreter (CHAIN_INTERPRET). */

constexpr uint32_t CH_MUL = 1, CH_SUB = 2, CH_DIV = 3, CH_ADD = 4, CH_SWAP = 6, CH_SAT = 7, CH_YUV = 8, CH_DIVC = 9,
                   CH_CASTI = 10, CH_CASTU = 11, CH_YUV601 = 12, CH_YUV2020 = 13;
#if defined(__CUDACC__)
__host__ __device__
#endif
constexpr uint32_t chain_of(uint32_t a = 0, uint32_t b = 0, uint32_t c = 0, uint32_t d = 0, uint32_t e = 0) {
    return a | (b << 4) | (c << 8) | (d << 12) | (e << 16);
}

}  // namespace fkb

#endif
