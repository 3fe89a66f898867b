/* Host side of the C ABI: validation, host-derived parameters, plan upload and launch.
 *
 * Replaces, for this path, the reference's compile-time lowering of a sender chain
 * (operation_model/iop_fuser.h:44-129, fused_operation.h), the batch builder
 * (batch_operations.h:178-208) and the launch site (executors.h:252-287).
 */
#include <cuda.h> /* CUtensorMap and the type of cuTensorMapEncodeTiled; the function itself is asked from the runtime */
#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>

#include <dlfcn.h>

#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <thread>
#include <deque>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <cmath>
#include <map>
#include <mutex>
#include <new>
#include <string>
#include <tuple>
#include <vector>

#include "fkb200.h"
#include "fkb_device.h"

namespace fkb {
cudaError_t launch_plan_kernel(uint32_t launch_class, uint32_t chain, const LaunchArgs& a, cudaStream_t stream);
bool chain_is_compiled(uint32_t chain);
}

using namespace fkb;

/* ------------------------------------------------------------------------------------ */
/* errors                                                                               */
/* ------------------------------------------------------------------------------------ */
static thread_local char g_last_error[512] = "";

static int fail(int status, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof g_last_error, fmt, ap);
    va_end(ap);
    return status;
}

/* Same wording as the reference's gpuErrchk (core/utils/utils.h:95-109). */
static int fail_cuda(cudaError_t e, const char* what, int line) {
    return fail(FKB_ERR_CUDA, "GPU Error: %s (%s) File: %s Line: %d", cudaGetErrorString(e), what, "fkb_host.cu", line);
}
#define FKB_CUDA(call)                                                   \
    do {                                                                 \
        const cudaError_t e__ = (call);                                  \
        if (e__ != cudaSuccess) return fail_cuda(e__, #call, __LINE__);  \
    } while (0)

/* Named ranges for profilers' timelines (the reference marks its tests the same way, tests/nvtx.h:18-104);
   without a tool attached a push or pop costs a few nanoseconds. */
struct NvtxRange {
    explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
    ~NvtxRange() { nvtxRangePop(); }
};

/* ------------------------------------------------------------------------------------ */
/* device memory: every allocation of the library goes through these, and is counted     */
/* ------------------------------------------------------------------------------------ */
static std::atomic<uint64_t> g_n_device_alloc{0}, g_n_device_free{0}, g_n_pinned_alloc{0}, g_n_lowered{0}, g_n_reused{0};

static cudaError_t device_alloc(void** p, size_t bytes) {
    g_n_device_alloc.fetch_add(1, std::memory_order_relaxed);
    return cudaMalloc(p, bytes);
}
static cudaError_t device_free(void* p) {
    g_n_device_free.fetch_add(1, std::memory_order_relaxed);
    return cudaFree(p);
}
static cudaError_t pinned_alloc(void** p, size_t bytes) {
    g_n_pinned_alloc.fetch_add(1, std::memory_order_relaxed);
    return cudaHostAlloc(p, bytes, cudaHostAllocDefault);
}

extern "C" FKB_API int fkb_debug_get_counters(fkb_debug_counters* out) {
    if (!out) return FKB_ERR_INVALID_ARGUMENT;
    out->device_allocations = g_n_device_alloc.load();
    out->device_frees = g_n_device_free.load();
    out->host_pinned_allocations = g_n_pinned_alloc.load();
    out->plans_lowered = g_n_lowered.load();
    out->plans_reused = g_n_reused.load();
    return FKB_OK;
}

/* ------------------------------------------------------------------------------------ */
/* plan object                                                                          */
/* ------------------------------------------------------------------------------------ */
struct fkb_plan {
    int device = -1;
    void* d_block = nullptr; /* one allocation: planes | seqs | ops | work-item table | status word */
    size_t d_bytes = 0;
    LaunchArgs args{};
    uint32_t launch_class = CLASS_GENERIC;
    uint32_t chain = CHAIN_INTERPRET;
    std::vector<fkb_resize_params> resize;
    fkb_plan_info info{};
};

/* What one plan needs in device memory, laid out for a single copy. */
struct HostImage {
    std::vector<DevPlane> planes;
    std::vector<DevSeq> seqs;
    std::vector<DevOp> ops;
    std::vector<uint32_t> item_start;
    std::vector<fkb_resize_params> resize;
    uint32_t launch_class = CLASS_GENERIC;
    uint32_t n_user_planes = 0;         /* planes of the description (a wide staged plane is several DevPlanes) */
    uint32_t chain = CHAIN_INTERPRET;   /* compiled chain shared by every sequence, or CHAIN_INTERPRET */
    uint32_t block_threads = BLOCK_THREADS;
    uint32_t total_items = 0;
    uint32_t max_seq_ops = 0;
    uint32_t staged_bytes = 0;          /* > 0: a STAGED class, this much shared memory per block */
    bool early_copies = false;          /* staged uchar3 classes: two table entries per block     */
    bool nv12_early = false;            /* staged NV12 class: NV12_ITEM_WORDS table words per block, with the rows to copy */
    size_t item_bytes() const { return early_copies ? 32 : nv12_early ? 16 * NV12_ITEM_WORDS : 16; }
    /* staged uchar3 classes, when every band can be one tiled copy: the tensor maps (one per distinct source image, row
       length and row count) and, per plane, the index of its map, its row bytes and its rows per tile */
    bool tiled_copies = false;
    std::vector<CUtensorMap> tmaps;
    struct PlaneTile { uint32_t map = 0, row_len = 0, rows = 0; };
    std::vector<PlaneTile> plane_tile;
    uint64_t output_pixels = 0;
    uint64_t algorithmic_bytes = 0;
    int n_constant_divisions = 0, n_ieee_divisions = 0;

    size_t off_planes() const { return 0; }
    size_t off_seqs() const { return planes.size() * sizeof(DevPlane); }
    size_t off_ops() const { return off_seqs() + seqs.size() * sizeof(DevSeq); }
    size_t off_items() const { return off_ops() + std::max<size_t>(ops.size(), 1) * sizeof(DevOp); }
    size_t off_status() const { return off_items() + (size_t)total_items * item_bytes(); }
    size_t off_tmaps() const { return (off_status() + 16 + 127) & ~(size_t)127; }
    size_t bytes() const { return tiled_copies ? off_tmaps() + tmaps.size() * TENSOR_MAP_BYTES : off_status() + 16; }

    /* One dense float3 -> float3 element-wise plane whose chain is long: how many work items ahead of its own a block
       prefetches into the L2 (LaunchArgs::prefetch_items), else 0. */
    uint32_t prefetch_items() const {
        if (launch_class != CLASS_FLAT_F32_F32 || planes.size() != 1 || seqs.size() != 1 || planes[0].n_segs != 1) return 0;
        uint64_t n_arith = 0;
        for (size_t k = 0; k < ops.size(); ++k) {
            if (ops[k].opcode == DEV_OP_REPEAT) {
                uint32_t count, period;
                std::memcpy(&count, &ops[k].p[0], 4); std::memcpy(&period, &ops[k].p[1], 4);
                n_arith += (uint64_t)count * period;
                k += period;
            } else ++n_arith;
        }
        if (n_arith < FLAT_PREFETCH_MIN_OPS || total_items <= FLAT_PREFETCH_ITEMS) return 0;
        return FLAT_PREFETCH_ITEMS;
    }

    /* The words behind a staged NV12 work item's entry (28 of 32 bits each): what the kernel's first two warps need to start
       the band tile's copies before the plane's descriptor has arrived.  The same arithmetic as body_nv12_staged: binary32
       product, floor, a second tap only where its weight is not zero and it is not clamped onto the first. */
    static void nv12_item_words(const DevPlane& dp, uint32_t local, uint32_t* w) {
        std::memset(w, 0, 4 * 4 * (NV12_ITEM_WORDS - 1));
        if (local >= dp.roi_items) return; /* store-only item */
        auto first_tap = [](int r, float f) { volatile float s = (float)r * f; return (int)std::floor(s); };
        const uint32_t g_lo = (uint32_t)dp.x1 / PX_PER_THREAD;
        const uint32_t n_groups = (uint32_t)dp.x2 / PX_PER_THREAD - g_lo + 1;
        const uint32_t band = local / dp.tiles_x, tile_x = local - band * dp.tiles_x, band_rows = dp.seg_pixels, gw = dp.gw;
        const int ya = dp.y1 + (int)(band * band_rows), yb = std::min(ya + (int)band_rows - 1, dp.y2);
        const int c_base = (int)(g_lo * PX_PER_THREAD + tile_x * 2 * gw);
        const int x_end = (int)std::min((g_lo + n_groups) * PX_PER_THREAD, (uint32_t)c_base + 2 * gw);
        const int rc0 = std::min(std::max(c_base, dp.x1), dp.x2), rc1 = std::max(std::min(x_end - 1, dp.x2), rc0);
        const int sx_first = dp.crop_x + first_tap(rc0 - dp.x1, dp.fx);
        const int sx_last = dp.crop_x + std::min(first_tap(rc1 - dp.x1, dp.fx) + 1, dp.crop_w - 1);
        const uint32_t byte0 = (uint32_t)sx_first & ~15u;
        const uint32_t row_len = std::min(((uint32_t)sx_last + 2u + 15u) & ~15u, dp.src_pitch) - byte0;
        const int l_first = dp.crop_y + first_tap(ya - dp.y1, dp.fy);
        const int l_last = dp.crop_y + std::min(first_tap(yb - dp.y1, dp.fy) + 1, dp.crop_h - 1);
        const int c_first = l_first >> 1;
        unsigned char* const luma_bits = reinterpret_cast<unsigned char*>(w + 12);
        unsigned char* const chroma_bits = reinterpret_cast<unsigned char*>(w + 20);
        auto mark = [&](int row) {
            const uint32_t a = (uint32_t)(row - l_first), b = (uint32_t)((row >> 1) - c_first);
            luma_bits[a >> 3] |= (unsigned char)(1u << (a & 7u));
            chroma_bits[b >> 3] |= (unsigned char)(1u << (b & 7u));
        };
        for (int y = ya; y <= yb; ++y) {
            volatile float s = (float)(y - dp.y1) * dp.fy;
            const int i0 = (int)std::floor(s);
            volatile float w1 = s - (float)i0;
            mark(dp.crop_y + i0);
            if (w1 != 0.0f) mark(dp.crop_y + std::min(i0 + 1, dp.crop_h - 1));
        }
        uint32_t n_luma = 0;
        for (int k = 0; k < 32; ++k) n_luma += (uint32_t)__builtin_popcount(luma_bits[k]);
        const uintptr_t luma = reinterpret_cast<uintptr_t>(dp.src) + (size_t)l_first * dp.src_pitch + byte0;
        const uintptr_t chroma = reinterpret_cast<uintptr_t>(dp.src) + (size_t)dp.src_pitch * dp.src_height + (size_t)c_first * dp.src_pitch + byte0;
        w[0] = (uint32_t)(luma & 0xFFFFFFFFu); w[1] = (uint32_t)((uint64_t)luma >> 32);
        w[2] = (uint32_t)(chroma & 0xFFFFFFFFu); w[3] = (uint32_t)((uint64_t)chroma >> 32);
        w[4] = dp.src_pitch; w[5] = row_len; w[6] = (uint32_t)(l_last - l_first + 1); w[7] = n_luma;
    }

    void serialize(unsigned char* dst) const {
        std::memcpy(dst + off_planes(), planes.data(), planes.size() * sizeof(DevPlane));
        std::memcpy(dst + off_seqs(), seqs.data(), seqs.size() * sizeof(DevSeq));
        if (!ops.empty()) std::memcpy(dst + off_ops(), ops.data(), ops.size() * sizeof(DevOp));
        /* work-item table: item_start holds the prefix sums of the items per plane */
        /* Blocks start in table order.  In a plan of several classes the planes that interpolate
           go first: their blocks take longest, and started last they would run alone at the end. */
        std::vector<size_t> order(planes.size());
        for (size_t i = 0; i < order.size(); ++i) order[i] = i;
        if (launch_class == CLASS_MIXED)
            std::stable_partition(order.begin(), order.end(), [&](size_t i) {
                const uint32_t c = planes[i].plane_class;
                return c == CLASS_RESIZE_U8_PLANAR || c == CLASS_RESIZE_U8_PACKED || c == CLASS_RESIZE_NV12_PACKED || c == CLASS_GENERIC ||
                       c == CLASS_RESIZE_U8_PLANAR_STAGED || c == CLASS_RESIZE_U8_PACKED_STAGED;
            });
        uint32_t* e = reinterpret_cast<uint32_t*>(dst + off_items());
        struct Item { uint32_t plane, local; double key; };
        std::vector<Item> table;
        table.reserve(total_items);
        for (size_t i : order)
            for (uint32_t l = 0, n = item_start[i + 1] - item_start[i]; l < n; ++l) table.push_back({(uint32_t)i, l, 0.0});
        if (launch_class == CLASS_MIXED) {
            /* Behind the interpolating planes, the items of the other sequences are spread evenly over the table (an item's
               place = its rank within its sequence / the sequence's size): blocks of a chain that is bound by instruction
               issue then run beside blocks of chains that are bound by memory, instead of alone at the end (four chains x 16
               images: 254.5 -> 250.9 us; spreading the interpolating planes as well: 260.5). */
            std::vector<uint64_t> size(seqs.size(), 0), rank(seqs.size(), 0);
            auto interpolates = [&](const Item& t) {
                const uint32_t c = planes[t.plane].plane_class;
                return c == CLASS_RESIZE_U8_PLANAR || c == CLASS_RESIZE_U8_PACKED || c == CLASS_RESIZE_NV12_PACKED || c == CLASS_GENERIC ||
                       c == CLASS_RESIZE_U8_PLANAR_STAGED || c == CLASS_RESIZE_U8_PACKED_STAGED;
            };
            for (const Item& t : table) ++size[planes[t.plane].seq];
            for (Item& t : table) {
                const uint32_t q = planes[t.plane].seq;
                t.key = interpolates(t) ? -1.0 : ((double)rank[q]++ + 0.5) / (double)size[q];
            }
            std::stable_sort(table.begin(), table.end(), [](const Item& a, const Item& b) { return a.key < b.key; });
        }
        for (const Item& t : table) {
            const size_t i = t.plane;
            const DevSeq& q = seqs[planes[i].seq];
            const DevPlane& dp = planes[i];
            for (uint32_t l = t.local, once = 0; once < 1; ++once, e += 4) {
                e[0] = (uint32_t)i; e[1] = l; e[2] = dp.seq | ((uint32_t)q.n_ops << 16); e[3] = (uint32_t)q.ops_begin;
                if (nv12_early) {
                    nv12_item_words(dp, l, e + 4);
                    e += 4 * (NV12_ITEM_WORDS - 1);
                    continue;
                }
                if (!early_copies) continue;
                /* second entry: what the band's bulk copies need (nothing for a store-only item) */
                e += 4;
                e[0] = e[1] = e[2] = e[3] = 0;
                if (dp.plane_class != CLASS_RESIZE_U8_PLANAR_STAGED && dp.plane_class != CLASS_RESIZE_U8_PACKED_STAGED) continue;
                if (l >= dp.roi_items) continue;
                const uint32_t n_rows = (uint32_t)(dp.y2 - dp.y1 + 1);
                const uint32_t ra = l * dp.tiles_x, rb = std::min(ra + dp.tiles_x, n_rows) - 1;
                const int first = (int)std::floor((float)ra * dp.fy);
                const int last = std::min((int)std::floor((float)rb * dp.fy) + 1, dp.crop_h - 1);
                const StagedSpan span = staged_span(dp.crop_x, dp.crop_w, dp.seg_pixels, (uint32_t)(dp.x2 - dp.x1 + 1), dp.fx);
                const uint32_t row_len = span.row_len;
                if (tiled_copies) { /* one tile of the plane's tensor map: its rows from `first` on, all of them whatever the band needs */
                    const PlaneTile& pt = plane_tile[i];
                    e[0] = pt.map; e[1] = 0; e[2] = pt.row_len * pt.rows;
                    e[3] = (span.row_first / 8u) | ((uint32_t)(dp.crop_y + first) << 16);
                    continue;
                }
                const uintptr_t src = reinterpret_cast<uintptr_t>(dp.src) + (size_t)(dp.crop_y + first) * dp.src_pitch + span.row_first;
                e[0] = (uint32_t)(src & 0xFFFFFFFFu); e[1] = (uint32_t)((uint64_t)src >> 32);
                e[2] = (uint32_t)(last - first + 1) | (row_len << 16); e[3] = dp.src_pitch;
            }
        }
        std::memset(dst + off_status(), 0, 16);
        if (tiled_copies) {
            static_assert(sizeof(CUtensorMap) == TENSOR_MAP_BYTES, "tensor map size");
            std::memcpy(dst + off_tmaps(), tmaps.data(), tmaps.size() * TENSOR_MAP_BYTES);
        }
    }
    LaunchArgs args_for(const unsigned char* d_base) const {
        LaunchArgs a{};
        a.planes = reinterpret_cast<const DevPlane*>(d_base + off_planes());
        a.seqs = reinterpret_cast<const DevSeq*>(d_base + off_seqs());
        a.ops = reinterpret_cast<const DevOp*>(d_base + off_ops());
        a.items = reinterpret_cast<const uint4*>(d_base + off_items());
        a.n_planes = (uint32_t)planes.size();
        a.total_items = total_items;
        a.max_seq_ops = max_seq_ops;
        a.block_threads = block_threads;
        a.staged_bytes = staged_bytes;
        a.nv12_early = nv12_early ? 1u : 0u;
        a.tiled_copies = tiled_copies ? 1u : 0u;
        a.tmaps = tiled_copies ? d_base + off_tmaps() : nullptr;
        a.wait_limit_us = FKB_DEFAULT_WAIT_LIMIT_US;
        a.status = reinterpret_cast<uint32_t*>(const_cast<unsigned char*>(d_base) + off_status());
        /* a single image: its descriptors ride in the kernel arguments, so that a block starts
           without a round trip to global memory */
        if (planes.size() == 1 && seqs.size() == 1 && ops.size() <= (size_t)INLINE_MAX_OPS && staged_bytes == 0) {
            a.inline_plane = 1;
            a.plane0 = planes[0];
            a.seq0 = seqs[0];
            for (size_t k = 0; k < ops.size(); ++k) a.ops0[k] = ops[k];
            a.prefetch_items = prefetch_items();
        }
        return a;
    }
};

/* ------------------------------------------------------------------------------------ */
/* host-derived parameters                                                              */
/* ------------------------------------------------------------------------------------ */

/* cxp::round (constexpr_libs/constexpr_cmath.h:119-130): add or subtract one half, truncate. */
static float round_half_away(float x) {
    return x > 0.0f ? static_cast<float>(static_cast<int>(x + 0.5f)) : static_cast<float>(static_cast<int>(x - 0.5f));
}

extern "C" FKB_API int fkb_derive_resize(int32_t sw, int32_t sh, int32_t dw, int32_t dh, int32_t mode,
                                 fkb_resize_params* out) {
    if (!out) return fail(FKB_ERR_INVALID_ARGUMENT, "fkb_derive_resize: out is NULL");
    if (sw <= 0 || sh <= 0 || dw <= 0 || dh <= 0)
        return fail(FKB_ERR_INVALID_ARGUMENT, "fkb_derive_resize: sizes must be positive (%d x %d -> %d x %d)", sw, sh,
                    dw, dh);
    int tw = dw, th = dh;
    if (mode == FKB_RESIZE_PRESERVE_AR || mode == FKB_RESIZE_PRESERVE_AR_RN_EVEN || mode == FKB_RESIZE_PRESERVE_AR_LEFT) {
        /* compute_target_size (resize.h:196-221): fit the height first, fall back to fitting
           the width when the scaled width overflows.  RN_EVEN rounds the fitted width down to an
           even number before the comparison, and the fitted height when the width is the limit. */
        volatile float scale = static_cast<float>(dh) / static_cast<float>(sh);
        volatile float scaled_w = scale * static_cast<float>(sw);
        tw = static_cast<int>(round_half_away(scaled_w));
        if (mode == FKB_RESIZE_PRESERVE_AR_RN_EVEN) tw -= tw % 2;
        if (tw > dw) {
            volatile float scale_w = static_cast<float>(dw) / static_cast<float>(sw);
            volatile float scaled_h = scale_w * static_cast<float>(sh);
            tw = dw;
            th = static_cast<int>(round_half_away(scaled_h));
            if (mode == FKB_RESIZE_PRESERVE_AR_RN_EVEN) th -= th % 2;
        }
        out->x1 = mode == FKB_RESIZE_PRESERVE_AR_LEFT ? 0 : (dw - tw) / 2; /* resize.h:132-133,150-151 */
        out->y1 = (dh - th) / 2;
        out->x2 = out->x1 + tw - 1;
        out->y2 = out->y1 + th - 1;
    } else if (mode == FKB_RESIZE_IGNORE_AR) {
        out->x1 = 0; out->y1 = 0; out->x2 = dw - 1; out->y2 = dh - 1;
    } else {
        return fail(FKB_ERR_INVALID_ARGUMENT, "fkb_derive_resize: mode %d is not a resize mode", mode);
    }
    /* resize.h:108-112 / :127-128,153-156: double quotient, double reciprocal, one narrowing */
    const double cfx = static_cast<double>(tw) / static_cast<double>(sw);
    const double cfy = static_cast<double>(th) / static_cast<double>(sh);
    out->fx = static_cast<float>(1.0 / cfx);
    out->fy = static_cast<float>(1.0 / cfy);
    out->target_width = tw;
    out->target_height = th;
    return FKB_OK;
}

/* computeDiscardedThreads + the scan of computeBestSolution (executors.h:176-242). */
extern "C" FKB_API int fkb_reference_block_size(uint32_t ax, uint32_t ay, uint32_t* bx, uint32_t* by) {
    if (!bx || !by || ax == 0 || ay == 0) return fail(FKB_ERR_INVALID_ARGUMENT, "fkb_reference_block_size: bad argument");
    static const uint32_t X[4] = {32, 64, 128, 256};
    static const uint32_t Y[2][4] = {{8, 4, 2, 1}, {6, 3, 3, 2}};
    uint32_t best = UINT32_MAX, bi = 0, bj = 0;
    bool done = false;
    for (uint32_t i = 0; i < 4 && !done; ++i) {
        for (uint32_t j = 0; j < 2 && !done; ++j) {
            const uint32_t mx = ax % X[i], my = ay % Y[j][i];
            const uint32_t idle_x = mx ? X[i] - mx : 0, idle_y = my ? Y[j][i] - my : 0;
            const uint32_t idle = idle_x * (my ? ay + Y[j][i] : ay) + idle_y * ax;
            if (idle < best) {
                best = idle; bi = i; bj = j;
                done = (idle == 0);
            }
        }
    }
    *bx = X[bi];
    *by = Y[bj][bi];
    return FKB_OK;
}

/* ------------------------------------------------------------------------------------ */
/* division by a plan-time constant                                                     */
/* ------------------------------------------------------------------------------------ */
/* Div<float3> is a true IEEE division in the reference (basic_ops/arithmetic.h:84).  Its
 * divisor is fixed when the plan is made, so the kernels may use
 *     q0 = RN(x * r),  e = x - p*q0 (one FMA, exact),  q = RN(q0 + e*r),   r = RN(1/p)
 * which costs three instructions, but only where it is PROVEN to return RN(x/p):
 *  (1) per divisor: the sequence is compared with x/p for every one of the 2^23 significands
 *      of x in [1, 2).  Multiplying x by a power of two multiplies every intermediate by the
 *      same power exactly, so this covers every x for which nothing under- or overflows;
 *  (2) per use: a range analysis of the sequence shows that the dividend is +0 or has
 *      2^-100 <= |x| <= 2^100 (with 2^-20 <= |p| <= 2^20 every intermediate is then a normal
 *      number or exactly representable), and that it cannot be -0 (the sequence would
 *      return +0).
 * Anything else keeps the IEEE division. */
static inline uint32_t float_bits(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }
static inline float bits_float(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }

#if defined(__x86_64__)
__attribute__((target("fma")))
#endif
static bool check_all_significands(float p) {
    const float r = 1.0f / p, np = -p;
    for (uint32_t m = 0; m < (1u << 23); ++m) {
        const float x = bits_float(0x3F800000u | m);
        const float q0 = x * r;
        const float e = __builtin_fmaf(np, q0, x);
        const float q = __builtin_fmaf(e, r, q0);
        if (float_bits(q) != float_bits(x / p)) return false;
    }
    return true;
}

static bool constant_division_is_exact(float p) {
    static std::mutex mu;
    static std::map<uint32_t, bool> cache;
#if defined(__x86_64__)
    if (!__builtin_cpu_supports("fma")) return false;
#endif
    const float a = std::fabs(p);
    if (!(a >= 0x1p-20f && a <= 0x1p20f)) return false; /* also rejects NaN, 0, inf */
    std::lock_guard<std::mutex> lock(mu);
    const auto it = cache.find(float_bits(p));
    if (it != cache.end()) return it->second;
    const bool ok = check_all_significands(p); /* about 10 ms, once per divisor value */
    if (cache.size() >= 4096) cache.clear();
    cache[float_bits(p)] = ok;
    return ok;
}

/* What is known about the values flowing through a sequence (all three channels together). */
struct ValueRange {
    bool known = false;   /* false: anything, including NaN and infinities                    */
    double absmax = 0;    /* |v| <= absmax                                                    */
    int nz_exp = 0;       /* v != 0  =>  |v| >= 2^nz_exp                                      */
    int grain = 0;        /* every v is an integer multiple of 2^grain                        */
    bool nonneg = true;   /* v >= 0                                                           */
    bool neg_zero = false;/* v may be -0                                                      */
    void check() { if (!(absmax < 1e37) || nz_exp < -120 || grain < -140) known = false; }
};

static int exp_of(float f) { return std::ilogb(std::fabs(f)); }

/* Applies one reference operation to the range; returns true when a division at this point
   may use the constant form. */
static bool advance_range(ValueRange& v, const fkb_op& op) {
    const float* p = op.p;
    bool fast = false;
    switch (op.opcode) {
        case FKB_OP_MUL: {
            if (!v.known) break;
            int emin = 1000; double amax = 0; bool neg = false;
            for (int c = 0; c < 3; ++c) {
                if (!std::isfinite(p[c]) || p[c] == 0.0f) { v.known = false; return false; }
                emin = std::min(emin, exp_of(p[c])); amax = std::max(amax, (double)std::fabs(p[c])); neg |= p[c] < 0;
            }
            v.absmax *= amax * 1.000001; v.nz_exp += emin; v.grain = v.nz_exp - 23;
            if (neg) { v.neg_zero = true; v.nonneg = false; }
            break;
        }
        case FKB_OP_ADD: case FKB_OP_SUB: {
            if (!v.known) break;
            int nz = 1000, grain = v.grain; double amax = 0; bool any_zero = false;
            for (int c = 0; c < 3; ++c) {
                if (!std::isfinite(p[c])) { v.known = false; return false; }
                if (p[c] == 0.0f) { any_zero = true; nz = std::min(nz, v.nz_exp); continue; }
                const int ep = exp_of(p[c]);
                /* RN(a +- p) != 0: either |a| < |p|/2 and the result is at least |p|/2, or a is a
                   multiple of ulp(|p|/2) and so is the exact sum */
                nz = std::min(nz, std::max(std::min(v.grain, ep - 23), ep - 24));
                grain = std::min(grain, ep - 23);
                amax = std::max(amax, (double)std::fabs(p[c]));
            }
            v.absmax += amax; v.nz_exp = nz; v.grain = grain; v.nonneg = false;
            v.neg_zero = v.neg_zero && any_zero;
            break;
        }
        case FKB_OP_DIV: {
            bool exact = true; int emax = -1000; double amin = 1e300; bool neg = false;
            for (int c = 0; c < 3; ++c) {
                if (!std::isfinite(p[c]) || p[c] == 0.0f) { v.known = false; return false; }
                exact = exact && constant_division_is_exact(p[c]);
                emax = std::max(emax, exp_of(p[c])); amin = std::min(amin, (double)std::fabs(p[c])); neg |= p[c] < 0;
            }
            if (!v.known) break;
            fast = exact && v.absmax <= 0x1p100 && v.nz_exp >= -100 && !v.neg_zero;
            v.absmax = v.absmax / amin * 1.000001; v.nz_exp = v.nz_exp - emax - 1; v.grain = v.nz_exp - 23;
            if (neg) { v.neg_zero = true; v.nonneg = false; }
            break;
        }
        case FKB_OP_SATURATE_CAST_U8:
            v = ValueRange{true, 255.0, 0, 0, true, false};
            break;
        case FKB_OP_CAST_I32: case FKB_OP_CAST_U32: /* bit patterns from here on; nothing follows */
            v.known = false;
            break;
        case FKB_OP_YUV_TO_RGB_BT709_FULL:
            /* integers times the matrix of color_conversion.h:143-146: the smallest non-zero
               coefficient is 0.1873, so every product and sum is a multiple of 2^-26 */
            if (v.known) v = ValueRange{true, 512.0, -26, -26, false, false};
            break;
        case FKB_OP_YUV_TO_RGB_BT601_FULL: case FKB_OP_YUV_TO_RGB_BT2020_FULL:
            /* the same with coefficients down to 0.16 and up to 2.02: multiples of 2^-26 below 1024 */
            if (v.known) v = ValueRange{true, 1024.0, -26, -26, false, false};
            break;
        default: /* CAST_F32, SWAP_RB: values unchanged */
            break;
    }
    v.check();
    return fast;
}

/* Bilinear interpolation (interpolation.h:92-95) of values in range v.  step_exp_x/y: floor(log2)
   of the smallest source step of any plane using the sequence, capped at 0: a non-zero weight is a
   multiple of ulp(source coordinate) >= 2^(step_exp - 23). */
static void advance_range_resize(ValueRange& v, int step_exp_x, int step_exp_y, bool preserve, const float* bg) {
    if (v.known) {
        const int gx = step_exp_x - 23, gy = step_exp_y - 23;
        v.nz_exp = v.nz_exp + gx + gy;              /* one product value*weight, if not zero     */
        if (!v.nonneg) v.nz_exp -= 23;              /* signed terms may cancel down to one grain */
        v.grain = v.nz_exp - 23;
        v.absmax *= 1.001;
    }
    if (preserve && v.known) {
        for (int c = 0; c < 3; ++c) {
            if (!std::isfinite(bg[c])) { v.known = false; break; }
            v.absmax = std::max(v.absmax, (double)std::fabs(bg[c]));
            if (bg[c] != 0.0f) { v.nz_exp = std::min(v.nz_exp, exp_of(bg[c])); v.grain = std::min(v.grain, exp_of(bg[c]) - 23); }
            if (bg[c] < 0.0f) v.nonneg = false;
            if (bg[c] == 0.0f && std::signbit(bg[c])) v.neg_zero = true;
        }
    }
    v.check();
}

/* The default value of a PRESERVE_AR resize after the operations that follow the geometry stage
 * (resize.h:84-86), in the reference's arithmetic: binary32, every operation rounded, true
 * division (this file is compiled without contraction). */
static float saturate_round_u8_host(float f) {
    if (f > 255.0f) return 255.0f;
    if (f < 0.0f) return 0.0f;
    return (float)(int)(f + 0.5f);
}
/* What cvt.rzi.s32.f32 / cvt.rzi.u32.f32 return (truncation; out-of-range values saturate, NaN gives 0). */
static int32_t cast_to_i32(float f) {
    if (!(f == f)) return 0;
    if (f >= 2147483648.0f) return INT32_MAX;
    if (f <= -2147483648.0f) return INT32_MIN;
    return (int32_t)f;
}
static uint32_t cast_to_u32(float f) {
    if (!(f > 0.0f)) return 0u;
    if (f >= 4294967296.0f) return UINT32_MAX;
    return (uint32_t)f;
}
static void background_after_ops(const fkb_sequence& s, int n_pre, float out[3]) {
    volatile float v[3] = {s.background[0], s.background[1], s.background[2]};
    for (int k = n_pre; k < s.n_ops; ++k) {
        const fkb_op& op = s.ops[k];
        switch (op.opcode) {
            case FKB_OP_MUL: for (int c = 0; c < 3; ++c) v[c] = v[c] * op.p[c]; break;
            case FKB_OP_SUB: for (int c = 0; c < 3; ++c) v[c] = v[c] - op.p[c]; break;
            case FKB_OP_DIV: for (int c = 0; c < 3; ++c) v[c] = v[c] / op.p[c]; break;
            case FKB_OP_ADD: for (int c = 0; c < 3; ++c) v[c] = v[c] + op.p[c]; break;
            case FKB_OP_SWAP_RB: { const float t = v[0]; v[0] = v[2]; v[2] = t; break; }
            case FKB_OP_SATURATE_CAST_U8: for (int c = 0; c < 3; ++c) v[c] = saturate_round_u8_host(v[c]); break;
            case FKB_OP_CAST_I32: for (int c = 0; c < 3; ++c) v[c] = bits_float((uint32_t)cast_to_i32(v[c])); break;
            case FKB_OP_CAST_U32: for (int c = 0; c < 3; ++c) v[c] = bits_float(cast_to_u32(v[c])); break;
            default: break; /* casts leave a float value unchanged; YUV conversion never follows a resize */
        }
    }
    out[0] = v[0]; out[1] = v[1]; out[2] = v[2];
}

/* Device form of a sequence's operations. */
static uint32_t chain_code_of(int dev_opcode) {
    switch (dev_opcode) {
        case FKB_OP_MUL: return CH_MUL;
        case FKB_OP_SUB: return CH_SUB;
        case FKB_OP_DIV: return CH_DIV;
        case FKB_OP_ADD: return CH_ADD;
        case FKB_OP_SWAP_RB: return CH_SWAP;
        case FKB_OP_SATURATE_CAST_U8: return CH_SAT;
        case FKB_OP_YUV_TO_RGB_BT709_FULL: return CH_YUV;
        case FKB_OP_YUV_TO_RGB_BT601_FULL: return CH_YUV601;
        case FKB_OP_YUV_TO_RGB_BT2020_FULL: return CH_YUV2020;
        case DEV_OP_DIV_BY_CONSTANT: return CH_DIVC;
        case FKB_OP_CAST_I32: return CH_CASTI;
        case FKB_OP_CAST_U32: return CH_CASTU;
        default: return 0;
    }
}

/* layouts that only the one-pixel-per-thread body reads, together with their conversion to RGB */
static bool read_converts(int f) { return f >= FKB_SRC_P010 && f <= FKB_SRC_UYVY; }

/* Lowers one sequence into `out`; Cast<uchar3,float3> is exact on values already held as float and
   leaves no device operation.  Returns the chain code of the operations after the geometry stage
   (CHAIN_INTERPRET when it does not fit eight nibbles). */
static uint32_t lower_ops(const fkb_sequence& s, int n_pre, int step_exp_x, int step_exp_y, std::vector<DevOp>& out,
                          int& dev_n_pre) {
    ValueRange v;
    const bool extras = s.border_mode != FKB_BORDER_NONE || s.deinterlace != FKB_DEINTERLACE_NONE || s.resize_mode >= FKB_GEOMETRY_WARP_AFFINE;
    if (s.src_format != FKB_SRC_F32X3 && !extras) v = ValueRange{true, 255.0, 0, 0, true, false};
    dev_n_pre = (int)out.size();
    uint32_t chain = 0;
    int chain_len = 0;
    for (int k = 0; k <= s.n_ops; ++k) {
        if (k == n_pre && s.resize_mode != FKB_RESIZE_NONE) {
            advance_range_resize(v, step_exp_x, step_exp_y, s.resize_mode >= FKB_RESIZE_PRESERVE_AR, s.background);
            if (extras) v.known = false;
            dev_n_pre = (int)out.size();
            chain = 0; chain_len = 0;
        }
        if (k == s.n_ops) break;
        const fkb_op& op = s.ops[k];
        if (k == 0 && read_converts(s.src_format)) { v.known = false; continue; } /* the read converts: nothing on the device's list */
        const bool fast = advance_range(v, op);
        if (op.opcode == FKB_OP_CAST_F32) continue;
        {
            const uint32_t code = chain_code_of(op.opcode == FKB_OP_DIV && fast ? DEV_OP_DIV_BY_CONSTANT : op.opcode);
            if (chain_len < 8 && chain != CHAIN_INTERPRET) chain |= code << (4 * chain_len++);
            else chain = CHAIN_INTERPRET;
        }
        DevOp o;
        o.opcode = op.opcode; o.p[0] = op.p[0]; o.p[1] = op.p[1]; o.p[2] = op.p[2];
        if (op.opcode == FKB_OP_DIV && fast) {
            DevOp r;
            o.opcode = DEV_OP_DIV_BY_CONSTANT;
            r.opcode = 0;
            for (int c = 0; c < 3; ++c) { o.p[c] = -op.p[c]; r.p[c] = 1.0f / op.p[c]; }
            out.push_back(o);
            out.push_back(r);
        } else {
            out.push_back(o);
        }
    }
    /* The same parameter for the three channels in every arithmetic operation of a compiled chain: its uniform variant,
       if that is compiled too (CHAIN_UNIFORM). */
    if (chain != CHAIN_INTERPRET && chain_len < 8 && chain_is_compiled(chain | CHAIN_UNIFORM)) {
        bool uniform = true;
        for (size_t k = (size_t)dev_n_pre; k < out.size(); ++k)
            uniform = uniform && std::memcmp(&out[k].p[0], &out[k].p[1], 4) == 0 && std::memcmp(&out[k].p[0], &out[k].p[2], 4) == 0;
        if (uniform) chain |= CHAIN_UNIFORM;
    }
    /* A long continuation that repeats one operation or a pair of them (the reference spells this
       StaticLoop, basic_ops/static_loop.h:22-44) runs as a counted loop on the device: the
       repeated part is stored once behind a header slot. */
    if (chain == CHAIN_INTERPRET || !chain_is_compiled(chain)) { /* up to eight operations that are no compiled chain are interpreted too */
        const size_t begin = (size_t)dev_n_pre;
        std::vector<DevOp> packed(out.begin() + begin, out.end());
        std::vector<DevOp> res;
        auto simple = [](const DevOp& o) { return o.opcode == FKB_OP_MUL || o.opcode == FKB_OP_SUB || o.opcode == FKB_OP_ADD; };
        auto same = [](const DevOp& x, const DevOp& y) { return std::memcmp(&x, &y, sizeof(DevOp)) == 0; };
        size_t i = 0;
        while (i < packed.size()) {
            size_t best_period = 0, best_count = 0;
            for (size_t period = 1; period <= 2; ++period) {
                if (i + period > packed.size()) break;
                bool ok = true;
                for (size_t q = 0; q < period; ++q) ok = ok && simple(packed[i + q]);
                if (!ok) continue;
                size_t count = 1;
                while (i + (count + 1) * period <= packed.size()) {
                    bool eq = true;
                    for (size_t q = 0; q < period; ++q) eq = eq && same(packed[i + q], packed[i + count * period + q]);
                    if (!eq) break;
                    ++count;
                }
                if (count * period >= 6 && count * period > best_count * best_period) { best_period = period; best_count = count; }
            }
            if (best_period) {
                DevOp head;
                head.opcode = DEV_OP_REPEAT;
                head.p[0] = bits_float((uint32_t)best_count); head.p[1] = bits_float((uint32_t)best_period); head.p[2] = 0.0f;
                res.push_back(head);
                for (size_t q = 0; q < best_period; ++q) res.push_back(packed[i + q]);
                i += best_count * best_period;
            } else {
                res.push_back(packed[i++]);
            }
        }
        if (res.size() < packed.size()) {
            out.resize(begin);
            out.insert(out.end(), res.begin(), res.end());
        }
    }
    return chain;
}

/* ------------------------------------------------------------------------------------ */
/* validation and lowering                                                              */
/* ------------------------------------------------------------------------------------ */
enum ValueType { VT_U8 = 0, VT_F32 = 1, VT_YUV8 = 2, VT_I32 = 3, VT_U32 = 4 };

static uint32_t src_pixel_bytes(int f) { return f == FKB_SRC_U8X3 ? 3u : f == FKB_SRC_F32X3 ? 12u : 1u; }
static bool is_yuv_source(int f) { return f >= FKB_SRC_NV12 && f <= FKB_SRC_UYVY; }

static bool is_yuv_conversion(int opcode) {
    return opcode == FKB_OP_YUV_TO_RGB_BT709_FULL || opcode == FKB_OP_YUV_TO_RGB_BT601_FULL || opcode == FKB_OP_YUV_TO_RGB_BT2020_FULL;
}
static uint32_t dst_pixel_bytes(int f) { return f == FKB_DST_U8X3_PACKED ? 3u : f == FKB_DST_F32_PLANAR3 ? 4u : 12u; }

/* Walks a sequence's operations with the value type the reference's templates would have
   (a mismatch there is a compile error; here it is FKB_ERR_INVALID_ARGUMENT). */
static int check_sequence(const fkb_sequence& s, int index, DevSeq& ds) {
    if (s.src_format < FKB_SRC_U8X3 || s.src_format > FKB_SRC_UYVY)
        return fail(FKB_ERR_INVALID_ARGUMENT, "sequence %d: unknown source format %d", index, s.src_format);
    if (s.dst_format < FKB_DST_F32X3_PACKED || s.dst_format > FKB_DST_U32X3_PACKED)
        return fail(FKB_ERR_INVALID_ARGUMENT, "sequence %d: unknown destination format %d", index, s.dst_format);
    if (s.resize_mode < FKB_RESIZE_NONE || s.resize_mode > FKB_GEOMETRY_WARP_PERSPECTIVE)
        return fail(FKB_ERR_INVALID_ARGUMENT, "sequence %d: unknown resize mode %d", index, s.resize_mode);
    if (s.border_mode < FKB_BORDER_NONE || s.border_mode > FKB_BORDER_REFLECT_101)
        return fail(FKB_ERR_INVALID_ARGUMENT, "sequence %d: unknown border mode %d", index, s.border_mode);
    if (s.deinterlace < FKB_DEINTERLACE_NONE || s.deinterlace > FKB_DEINTERLACE_LINEAR_ODD)
        return fail(FKB_ERR_INVALID_ARGUMENT, "sequence %d: unknown deinterlace mode %d", index, s.deinterlace);
    if ((s.border_mode != FKB_BORDER_NONE || s.deinterlace != FKB_DEINTERLACE_NONE) && is_yuv_source(s.src_format))
        return fail(FKB_ERR_UNSUPPORTED, "sequence %d: BorderReader and Deinterlace over a YUV read are not on this path", index);
    if (s.border_mode != FKB_BORDER_NONE && s.deinterlace != FKB_DEINTERLACE_NONE)
        return fail(FKB_ERR_UNSUPPORTED, "sequence %d: BorderReader together with Deinterlace is not on this path", index);
    if (s.n_ops < 0 || s.n_ops > 4096) return fail(FKB_ERR_INVALID_ARGUMENT, "sequence %d: n_ops %d outside [0, 4096]", index, s.n_ops);
    if (s.n_ops > 0 && !s.ops) return fail(FKB_ERR_INVALID_ARGUMENT, "sequence %d: ops is NULL", index);
    const int n_pre = s.resize_mode == FKB_RESIZE_NONE ? 0 : s.n_pre_ops;
    if (n_pre < 0 || n_pre > s.n_ops)
        return fail(FKB_ERR_INVALID_ARGUMENT, "sequence %d: n_pre_ops %d outside [0, n_ops]", index, s.n_pre_ops);

    ValueType t = s.src_format == FKB_SRC_U8X3 ? VT_U8 : s.src_format == FKB_SRC_F32X3 ? VT_F32 : VT_YUV8;
    if (s.deinterlace != FKB_DEINTERLACE_NONE) t = VT_F32; /* Deinterlace returns float3 (deinterlace.h:47-50) */
    bool pre_only_casts = true, pre_is_yuv = (n_pre == 1);
    int yuv_opcode = 0;
    for (int k = 0; k <= s.n_ops; ++k) {
        if (k == n_pre && s.resize_mode != FKB_RESIZE_NONE) t = VT_F32; /* Interpolate returns float (interpolation.h:55-57) */
        if (k == s.n_ops) break;
        const int oc = s.ops[k].opcode;
        if (k < n_pre) {
            if (oc != FKB_OP_CAST_F32) pre_only_casts = false;
            if (!is_yuv_conversion(oc)) pre_is_yuv = false;
            else yuv_opcode = oc;
        }
        if (t == VT_I32 || t == VT_U32)
            return fail(FKB_ERR_INVALID_ARGUMENT, "sequence %d op %d: nothing but the receiver may follow a cast to int3 / uint3", index, k);
        switch (oc) {
            case FKB_OP_CAST_I32: case FKB_OP_CAST_U32:
                if (t != VT_F32) return fail(FKB_ERR_INVALID_ARGUMENT, "sequence %d op %d: Cast<float3,int3|uint3> needs a float value", index, k);
                if (k < n_pre) return fail(FKB_ERR_INVALID_ARGUMENT, "sequence %d op %d: an integer cast cannot precede the interpolation", index, k);
                t = oc == FKB_OP_CAST_I32 ? VT_I32 : VT_U32;
                break;
            case FKB_OP_MUL: case FKB_OP_SUB: case FKB_OP_DIV: case FKB_OP_ADD:
                if (t != VT_F32) return fail(FKB_ERR_INVALID_ARGUMENT, "sequence %d op %d: arithmetic on a non-float value (add a Cast first)", index, k);
                break;
            case FKB_OP_CAST_F32:
                if (t == VT_YUV8) return fail(FKB_ERR_INVALID_ARGUMENT, "sequence %d op %d: Cast on packed YUV is not part of this path", index, k);
                t = VT_F32;
                break;
            case FKB_OP_SWAP_RB: break;
            case FKB_OP_SATURATE_CAST_U8:
                if (t != VT_F32) return fail(FKB_ERR_INVALID_ARGUMENT, "sequence %d op %d: SaturateCast<float3,uchar3> needs a float value", index, k);
                t = VT_U8;
                break;
            case FKB_OP_YUV_TO_RGB_BT709_FULL: case FKB_OP_YUV_TO_RGB_BT601_FULL: case FKB_OP_YUV_TO_RGB_BT2020_FULL:
                if (t != VT_YUV8) return fail(FKB_ERR_INVALID_ARGUMENT, "sequence %d op %d: ConvertYUVToRGB needs the value read by ReadYUV", index, k);
                t = VT_F32;
                break;
            default:
                return fail(FKB_ERR_INVALID_ARGUMENT, "sequence %d op %d: unknown opcode %d", index, k, oc);
        }
    }
    if (read_converts(s.src_format) && (s.n_ops < 1 || !is_yuv_conversion(s.ops[0].opcode) || (s.resize_mode != FKB_RESIZE_NONE && n_pre < 1)))
        return fail(FKB_ERR_UNSUPPORTED, "sequence %d: a P010 / P210 / Y210 / UYVY read must be followed at once by its conversion to RGB", index);
    const bool dst_u8 = s.dst_format == FKB_DST_U8X3_PACKED;
    const ValueType want = dst_u8 ? VT_U8 : s.dst_format == FKB_DST_I32X3_PACKED ? VT_I32 : s.dst_format == FKB_DST_U32X3_PACKED ? VT_U32 : VT_F32;
    if (want != (t == VT_YUV8 ? VT_U8 : t)) {
        static const char* const names[] = {"uchar", "float", "uchar", "int", "uint"};
        return fail(FKB_ERR_INVALID_ARGUMENT, "sequence %d: chain ends in a %s value but the receiver writes %s", index,
                    names[t], names[want]);
    }

    ds.src_format = s.src_format; ds.dst_format = s.dst_format; ds.resize_mode = s.resize_mode;
    /* NV21 is NV12 with the two chroma bytes exchanged (color_conversion.h:347-359): the kernels read it as NV12
       and swap the pair of every tap */
    ds.swap_uv = s.src_format == FKB_SRC_NV21 ? 1u : 0u;
    if (s.src_format == FKB_SRC_NV21) ds.src_format = FKB_SRC_NV12;
    /* int3 / uint3 pixels are twelve bytes like float3 and their values travel as bit patterns: the
       kernels store them through the float3 receiver */
    if (want == VT_I32 || want == VT_U32) ds.dst_format = FKB_DST_F32X3_PACKED;
    ds.n_ops = s.n_ops; ds.n_pre = n_pre; ds.ops_begin = 0; ds.chain = CHAIN_INTERPRET;
    const bool read_back_extras = s.border_mode != FKB_BORDER_NONE || s.deinterlace != FKB_DEINTERLACE_NONE ||
                                  s.resize_mode >= FKB_GEOMETRY_WARP_AFFINE;
    ds.border_mode = s.border_mode; ds.deinterlace = s.deinterlace;
    for (int c = 0; c < 3; ++c) ds.border_value[c] = s.border_value[c];
    for (int k = 0; k < 9; ++k) ds.transform[k] = s.transform[k];
    ds.yuv_kind = 0; ds.yuv_shift = 0;
    if (read_converts(s.src_format)) {
        const int oc = s.ops[0].opcode;
        ds.yuv_kind = oc == FKB_OP_YUV_TO_RGB_BT709_FULL ? PRE_YUV_BT709 : oc == FKB_OP_YUV_TO_RGB_BT601_FULL ? PRE_YUV_BT601 : PRE_YUV_BT2020;
        ds.yuv_shift = s.src_format == FKB_SRC_UYVY ? 0u : 6u;
    }
    /* BorderReader, Deinterlace, Warping and the layouts whose read converts run in the one-pixel-per-thread body only */
    ds.pre_kind = (read_back_extras || read_converts(s.src_format)) ? PRE_GENERAL
                  : (n_pre == 0 || pre_only_casts) ? PRE_IDENTITY
                  : !pre_is_yuv ? PRE_GENERAL
                  : yuv_opcode == FKB_OP_YUV_TO_RGB_BT709_FULL ? PRE_YUV_BT709
                  : yuv_opcode == FKB_OP_YUV_TO_RGB_BT601_FULL ? PRE_YUV_BT601 : PRE_YUV_BT2020;
    ds.bg[0] = s.background[0]; ds.bg[1] = s.background[1]; ds.bg[2] = s.background[2]; ds.one = 1.0f;
    background_after_ops(s, n_pre, ds.bg_out);
    return FKB_OK;
}

/* STAGED classes: how a plane's region of interest is cut into bands whose source footprint
 * fits the shared-memory stage.  Source rows are found with the arithmetic the kernel uses
 * (binary32 product of the row index and fy, floor: resize.h:183-194, interpolation.h:66-67). */
struct StagedTiling {
    bool ok = false;
    uint32_t band_rows = 0, gw = 0, rs = 0, n_bands = 0, stage_bytes = 0;
    uint32_t row_len = 0, src_rows = 0; /* bytes of a staged row, and the most rows any band of the plane stages */
};
static int staged_src_row(int r, float fy) { return (int)std::floor((float)r * fy); }

static bool region_empty(const DevPlane& dp) { return dp.x2 < dp.x1 || dp.y2 < dp.y1; }

static StagedTiling staged_tiling(const DevPlane& dp, uint32_t block_threads, uint32_t band_pixels = STAGED_BAND_PIXELS) {
    StagedTiling t;
    if (region_empty(dp)) { /* nothing to interpolate: store-only items alone */
        t.ok = true; t.gw = block_threads; t.rs = 1;
        return t;
    }
    const uint32_t g_lo = (uint32_t)dp.x1 / PX_PER_THREAD;
    const uint32_t n_groups = (uint32_t)dp.x2 / PX_PER_THREAD - g_lo + 1;
    const uint32_t n_rows = (uint32_t)(dp.y2 - dp.y1 + 1);
    const uint32_t pairs = n_groups * (PX_PER_THREAD / 2); /* threads across: each owns two columns */
    if (pairs > block_threads) return t;
    if ((reinterpret_cast<uintptr_t>(dp.src) % 16) != 0 || (dp.src_pitch % 16) != 0) return t;
    const StagedSpan span = staged_span(dp.crop_x, dp.crop_w, dp.seg_pixels, (uint32_t)(dp.x2 - dp.x1 + 1), dp.fx);
    const uint32_t row_len = span.row_len;
    if (span.row_first + row_len > dp.src_pitch) return t; /* never reads past the end of a row */
    /* the kernel reads whole words around the last tap: 16 spare bytes behind the last row */
    const uint32_t max_src_rows = (STAGED_MAX_STAGE_BYTES - 16) / row_len;
    if (max_src_rows < 2) return t;
    t.gw = pairs;
    t.rs = block_threads / pairs;
    auto worst_rows = [&](uint32_t band) {
        uint32_t worst = 0;
        for (uint32_t a = 0; a < n_rows; a += band) {
            const uint32_t b = std::min(a + band, n_rows) - 1;
            const int first = staged_src_row((int)a, dp.fy);
            const int last = std::min(staged_src_row((int)b, dp.fy) + 1, dp.crop_h - 1);
            worst = std::max(worst, (uint32_t)(last - first + 1));
        }
        return worst;
    };
    /* Height limit: STAGED_MAX_ROWS rows, and about STAGED_BAND_PIXELS output pixels, so that a wide
       region is cut into more, shorter bands (their copies and arithmetic overlap across the blocks
       of an SM) while a narrow one stays in one block. */
    const uint32_t by_pixels = std::max<uint32_t>(t.rs, (band_pixels / (2u * pairs) + t.rs - 1) / t.rs * t.rs);
    uint32_t band = std::min<uint32_t>(std::min<uint32_t>(STAGED_MAX_ROWS, by_pixels), n_rows);
    {   /* first guess from the step, then exact */
        const double guess = ((double)max_src_rows - 2.0) / std::max((double)dp.fy, 1e-6) + 1.0;
        if (guess < (double)band) band = (uint32_t)std::max(1.0, guess);
    }
    while (band > 1 && worst_rows(band) > max_src_rows) --band;
    if (worst_rows(band) > max_src_rows) return t;
    /* Bands of equal height, in whole rounds of the row slots: 44 rows that fit one band are one
       band (not 40 + 4, each paying a block's start-up), 224 rows under a limit of 64 are 4 x 56. */
    {
        const uint32_t n_bands = (n_rows + band - 1) / band;
        uint32_t even = (n_rows + n_bands - 1) / n_bands;
        even = (even + t.rs - 1) / t.rs * t.rs;
        if (even <= STAGED_MAX_ROWS && worst_rows(even) <= max_src_rows) band = even;
        else if (band > t.rs) band -= band % t.rs;
    }
    t.band_rows = band;
    t.n_bands = (n_rows + band - 1) / band;
    t.row_len = row_len;
    t.src_rows = worst_rows(band);
    t.stage_bytes = t.src_rows * row_len + 16;
    t.ok = true;
    return t;
}

/* cuTensorMapEncodeTiled, asked from the runtime so that the library does not link the driver; null where there is no
   driver (a build box without a GPU). */
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult status = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &status) != cudaSuccess ||
            status != cudaDriverEntryPointSuccess) {
            (void)cudaGetLastError();
            p = nullptr;
        }
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

/* The tensor maps of a plan whose staged planes are one band each (a batch of small planes) and can all take the band's
   source rows as one tile: the image as rows of eight-byte elements (a tile starts at an even element, i.e. on a
   16-byte boundary, as the rows of the per-row copies do), box = the plane's staged row bytes x its band's rows.  A
   tile that reaches below the image is filled with zeros there.  One instruction by one thread then replaces one bulk
   copy per row, each of which costs about ten instructions of the warp that issues them: 8190 crops into 60 x 60 planes
   64.3 M -> 62.4 M warp instructions, 88.1 -> 86.0 us on the same GPU.  Planes of several bands keep the per-row copies: a
   map's box has one height, the most rows any band of the plane needs, so the other bands would fetch a row or two they
   do not use (1024 crops into 224 x 224: 152.7 us per row, 154.5 tiled).  False when a plane does not qualify or there is no
   driver: the plan then copies row by row. */
static bool build_tensor_maps(HostImage& img, const std::vector<StagedTiling>& st, const std::vector<uint32_t>& kept_items) {
#ifdef FKB_CHECK_BOUNDS
    (void)img; (void)st; (void)kept_items;
    return false; /* the checked build copies row by row, each row checked against the plane */
#else
    const EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) return false;
    struct Key {
        const uint8_t* src; uint32_t pitch, rows, row_len, box_rows;
        bool operator<(const Key& o) const { return std::tie(src, pitch, rows, row_len, box_rows) < std::tie(o.src, o.pitch, o.rows, o.row_len, o.box_rows); }
    };
    std::map<Key, uint32_t> seen;
    std::vector<CUtensorMap> maps;
    std::vector<HostImage::PlaneTile> tiles(img.planes.size());
    for (size_t i = 0; i < img.planes.size(); ++i) {
        if (kept_items[i] != 0 || region_empty(img.planes[i])) continue;
        if (st[i].n_bands > 1) return false;
        const DevPlane& dp = img.planes[i];
        const uint32_t src_rows_total = source_rows(FKB_SRC_U8X3, dp.src_height);
        if (st[i].row_len == 0 || st[i].row_len > TILED_MAX_ROW_BYTES || st[i].src_rows == 0 || st[i].src_rows > TILED_MAX_ROWS) return false;
        if (dp.src_pitch / 8u > 0xFFFFu || (uint32_t)dp.crop_y + (uint32_t)dp.crop_h > 0xFFFFu || src_rows_total == 0) return false;
        const Key key{dp.src, dp.src_pitch, src_rows_total, st[i].row_len, st[i].src_rows};
        auto it = seen.find(key);
        if (it == seen.end()) {
            CUtensorMap m;
            const cuuint64_t dims[2] = {dp.src_pitch / 8u, src_rows_total};
            const cuuint64_t strides[1] = {dp.src_pitch};
            const cuuint32_t box[2] = {st[i].row_len / 8u, st[i].src_rows};
            const cuuint32_t elem[2] = {1, 1};
            if (encode(&m, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<uint8_t*>(dp.src), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                       CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
                return false;
            it = seen.emplace(key, (uint32_t)maps.size()).first;
            maps.push_back(m);
        }
        tiles[i].map = it->second; tiles[i].row_len = st[i].row_len; tiles[i].rows = st[i].src_rows;
    }
    if (maps.empty()) return false;
    img.tmaps = std::move(maps);
    img.plane_tile = std::move(tiles);
    return true;
#endif
}

/* Staged NV12: bands of rows times tiles of columns; the luma and chroma rows between a band's
 * first and last tap, over the tile's byte range, must fit the stage. */
struct Nv12Tiling {
    bool ok = false;
    uint32_t band_rows = 0, gw = 0, rs = 0, tiles_x = 0, n_bands = 0, stage_bytes = 0;
};
static Nv12Tiling nv12_staged_tiling(const DevPlane& dp, uint32_t block_threads) {
    Nv12Tiling t;
    if (region_empty(dp)) { /* nothing to interpolate: store-only items alone */
        t.ok = true; t.gw = block_threads; t.rs = 1; t.tiles_x = 1;
        return t;
    }
    if ((reinterpret_cast<uintptr_t>(dp.src) % 16) != 0 || (dp.src_pitch % 16) != 0) return t;
    const uint32_t g_lo = (uint32_t)dp.x1 / PX_PER_THREAD;
    const uint32_t n_groups = (uint32_t)dp.x2 / PX_PER_THREAD - g_lo + 1;
    const uint32_t n_rows = (uint32_t)(dp.y2 - dp.y1 + 1);
    const uint32_t pairs = n_groups * (PX_PER_THREAD / 2);
    t.tiles_x = (pairs + block_threads - 1) / block_threads;
    t.gw = (pairs + t.tiles_x - 1) / t.tiles_x;
    t.rs = block_threads / t.gw;
    /* widest byte range of any column tile */
    uint32_t row_len = 0;
    for (uint32_t tx = 0; tx < t.tiles_x; ++tx) {
        const int c_base = (int)(g_lo * PX_PER_THREAD + tx * 2 * t.gw);
        const int x_end = (int)std::min((g_lo + n_groups) * PX_PER_THREAD, (uint32_t)c_base + 2 * t.gw);
        const int rc0 = std::min(std::max(c_base, dp.x1), dp.x2), rc1 = std::max(std::min(x_end - 1, dp.x2), rc0);
        const int sx_first = dp.crop_x + staged_src_row(rc0 - dp.x1, dp.fx);
        const int sx_last = dp.crop_x + std::min(staged_src_row(rc1 - dp.x1, dp.fx) + 1, dp.crop_w - 1);
        const uint32_t byte0 = (uint32_t)sx_first & ~15u;
        row_len = std::max(row_len, std::min(((uint32_t)sx_last + 2u + 15u) & ~15u, dp.src_pitch) - byte0);
    }
    /* Per output row, as the kernel finds them (binary32 product, floor, weight of the second tap): the source row
       of the first vertical tap and whether the second tap is read at all (a weight of exactly zero is skipped). */
    std::vector<int> tap0(n_rows);
    std::vector<unsigned char> second(n_rows);
    for (uint32_t r = 0; r < n_rows; ++r) {
        volatile float s = (float)r * dp.fy;
        const int i0 = (int)std::floor(s);
        volatile float w1 = s - (float)i0;
        tap0[r] = dp.crop_y + i0;
        second[r] = w1 != 0.0f && i0 + 1 <= dp.crop_h - 1 ? 1 : 0; /* a clamped second tap is the first tap's row */
    }
    /* Rows a band must hold: the distinct luma rows and the distinct chroma rows its taps read (only those are
       copied and they are packed); `span` is the distance between its first and last luma row, which sizes the
       kernel's row-flag arrays. */
    auto worst = [&](uint32_t band, uint32_t& span) {
        uint32_t rows = 0;
        span = 0;
        for (uint32_t a = 0; a < n_rows; a += band) {
            const uint32_t b = std::min(a + band, n_rows) - 1;
            const int first = dp.crop_y + staged_src_row((int)a, dp.fy);
            const int last = dp.crop_y + std::min(staged_src_row((int)b, dp.fy) + 1, dp.crop_h - 1);
            uint32_t n_l = 0, n_c = 0;
            int last_l = -1, last_c = -1;
            for (uint32_t r = a; r <= b; ++r) {
                for (int k = 0; k <= (int)second[r]; ++k) { /* rows come in non-decreasing order */
                    const int l = tap0[r] + k;
                    if (l > last_l) { ++n_l; last_l = l; }
                    if ((l >> 1) > last_c) { ++n_c; last_c = l >> 1; }
                }
            }
            rows = std::max(rows, n_l + n_c);
            span = std::max(span, (uint32_t)(last - first + 1));
        }
        return rows;
    };
    uint32_t band = std::min<uint32_t>(STAGED_MAX_ROWS, n_rows), span = 0;
    auto too_big = [&](uint32_t b) { const uint32_t rows = worst(b, span); return rows * row_len > NV12_MAX_STAGE_BYTES || rows > 250u || span > NV12_MAX_SPAN; };
    while (band > 1 && too_big(band)) --band;
    if (too_big(band)) return t;
    if (band > t.rs) band -= band % t.rs;
    t.band_rows = band;
    t.n_bands = (n_rows + band - 1) / band;
    t.stage_bytes = worst(band, span) * row_len;
    t.ok = true;
    return t;
}

static bool aligned(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

static int lower(const fkb_plan_desc* d, HostImage& img) {
    if (!d) return fail(FKB_ERR_INVALID_ARGUMENT, "plan description is NULL");
    if (!d->sequences || d->n_sequences <= 0) return fail(FKB_ERR_INVALID_ARGUMENT, "plan has no sequences");
    if (d->n_sequences > 65535) return fail(FKB_ERR_INVALID_ARGUMENT, "plan has more than 65535 sequences");
    if (!d->planes || d->n_planes <= 0) return fail(FKB_ERR_INVALID_ARGUMENT, "plan has no planes (batch of 0)");

    img.seqs.resize(d->n_sequences);
    for (int s = 0; s < d->n_sequences; ++s) {
        const int rc = check_sequence(d->sequences[s], s, img.seqs[s]);
        if (rc) return rc;
    }
    /* smallest source step of any plane of a sequence, as floor(log2), capped at 0 */
    std::vector<int> step_exp_x(d->n_sequences, 0), step_exp_y(d->n_sequences, 0);

    img.planes.resize(d->n_planes);
    img.n_user_planes = (uint32_t)d->n_planes;
    img.resize.assign(d->n_planes, fkb_resize_params{});
    img.item_start.assign((size_t)d->n_planes + 1, 0);
    uint64_t total = 0;
    bool same_groups = false;
    uint32_t first_groups = 0;
    uint32_t common_class = CLASS_MIXED;
    for (int i = 0; i < d->n_planes; ++i) {
        const fkb_plane& p = d->planes[i];
        if (p.sequence < 0 || p.sequence >= d->n_sequences)
            return fail(FKB_ERR_INVALID_ARGUMENT, "plane %d: sequence index %d outside [0, %d)", i, p.sequence, d->n_sequences);
        const DevSeq& s = img.seqs[p.sequence];
        const bool is_default = (p.flags & FKB_PLANE_DEFAULT_VALUE) != 0; /* reads the default value, never its image */
        if (p.flags & ~FKB_PLANE_DEFAULT_VALUE) return fail(FKB_ERR_INVALID_ARGUMENT, "plane %d: unknown flag bits 0x%x", i, p.flags);
        if (!p.dst || (!p.src && !is_default)) return fail(FKB_ERR_INVALID_ARGUMENT, "plane %d: null image pointer", i);
        if (p.dst_width == 0 || p.dst_height == 0 || (!is_default && (p.src_width == 0 || p.src_height == 0)))
            return fail(FKB_ERR_INVALID_ARGUMENT, "plane %d: zero-sized image", i);
        if (p.src_width > (1u << 24) || p.src_height > (1u << 24) || p.dst_width > (1u << 24) || p.dst_height > (1u << 24))
            return fail(FKB_ERR_INVALID_ARGUMENT, "plane %d: image side beyond 2^24", i);
        const uint32_t spx = src_pixel_bytes(s.src_format), dpx = dst_pixel_bytes(s.dst_format);
        if (!is_default) {
            const uint64_t src_row = source_row_bytes(s.src_format, p.src_width);
            if (p.src_pitch < src_row)
                return fail(FKB_ERR_INVALID_ARGUMENT, "plane %d: source pitch %u is less than a row of %llu bytes", i, p.src_pitch, (unsigned long long)src_row);
            if ((uint64_t)p.src_pitch * p.src_height * 2 > 0xFFFFFFFFull)
                return fail(FKB_ERR_INVALID_ARGUMENT, "plane %d: source image beyond 2 GiB", i);
            const bool padded = s.border_mode != FKB_BORDER_NONE; /* BorderReader below the Crop: the rect may reach beyond the image */
            if (p.crop_width <= 0 || p.crop_height <= 0 || p.crop_width > (1 << 24) || p.crop_height > (1 << 24) ||
                (padded ? (p.crop_x < -(1 << 24) || p.crop_y < -(1 << 24) || p.crop_x > (1 << 24) || p.crop_y > (1 << 24))
                        : (p.crop_x < 0 || p.crop_y < 0 || (uint64_t)p.crop_x + (uint64_t)p.crop_width > p.src_width ||
                           (uint64_t)p.crop_y + (uint64_t)p.crop_height > p.src_height)))
                return fail(FKB_ERR_INVALID_ARGUMENT, "plane %d: crop rect (%d,%d,%d,%d) outside its %ux%u image", i, p.crop_x, p.crop_y, p.crop_width, p.crop_height, p.src_width, p.src_height);
            if (s.resize_mode == FKB_RESIZE_NONE && ((uint32_t)p.crop_width != p.dst_width || (uint32_t)p.crop_height != p.dst_height))
                return fail(FKB_ERR_INVALID_ARGUMENT, "plane %d: without a resize the output (%ux%u) must have the size of the crop (%dx%d)", i, p.dst_width, p.dst_height, p.crop_width, p.crop_height);
            if (s.src_format == FKB_SRC_F32X3 && (!aligned(p.src, 4) || p.src_pitch % 4))
                return fail(FKB_ERR_INVALID_ARGUMENT, "plane %d: float source must be 4-byte aligned", i);
            if (read_converts(s.src_format) && (!aligned(p.src, 8) || p.src_pitch % 8))
                return fail(FKB_ERR_INVALID_ARGUMENT, "plane %d: a P010 / P210 / Y210 / UYVY image and its pitch must be 8-byte aligned", i);
        }
        if (p.dst_pitch < (uint64_t)p.dst_width * dpx)
            return fail(FKB_ERR_INVALID_ARGUMENT, "plane %d: destination pitch %u is less than a row of %llu bytes", i, p.dst_pitch, (unsigned long long)p.dst_width * dpx);
        if (s.dst_format != FKB_DST_U8X3_PACKED && (!aligned(p.dst, 4) || p.dst_pitch % 4 || p.dst_channel_stride % 4))
            return fail(FKB_ERR_INVALID_ARGUMENT, "plane %d: float destination must be 4-byte aligned", i);
        if (s.dst_format == FKB_DST_F32_PLANAR3 && p.dst_channel_stride < (uint64_t)p.dst_pitch * (p.dst_height - 1) + (uint64_t)p.dst_width * 4)
            return fail(FKB_ERR_INVALID_ARGUMENT, "plane %d: channel stride %u overlaps the channel plane", i, p.dst_channel_stride);

        DevPlane& dp = img.planes[i];
        std::memset(&dp, 0, sizeof dp);
        dp.src = static_cast<const uint8_t*>(p.src);
        dp.dst = static_cast<uint8_t*>(p.dst);
        dp.src_pitch = p.src_pitch; dp.src_height = p.src_height;
        dp.crop_x = p.crop_x; dp.crop_y = p.crop_y; dp.crop_w = p.crop_width; dp.crop_h = p.crop_height;
        dp.dst_w = p.dst_width; dp.dst_h = p.dst_height; dp.dst_pitch = p.dst_pitch; dp.dst_cstride = p.dst_channel_stride;
        dp.seq = (uint32_t)p.sequence;
        dp.fx = dp.fy = 1.0f;
        dp.x2 = (int32_t)p.dst_width - 1; dp.y2 = (int32_t)p.dst_height - 1;
        if (is_default) {
            /* every element is the default value: an empty region of interest, store-only work; the image is never read */
            dp.src = nullptr; dp.src_pitch = 0; dp.src_height = 0;
            dp.crop_x = dp.crop_y = 0; dp.crop_w = dp.crop_h = 1;
            dp.x1 = 0; dp.y1 = 0; dp.x2 = -1; dp.y2 = -1;
        } else if (s.resize_mode >= FKB_GEOMETRY_WARP_AFFINE) {
            /* Warping: every output element is computed (inside the source or 0); no host-derived factors */
        } else if (s.resize_mode != FKB_RESIZE_NONE) {
            fkb_resize_params& rp = img.resize[i];
            const int rc = fkb_derive_resize(p.crop_width, p.crop_height, (int32_t)p.dst_width, (int32_t)p.dst_height, s.resize_mode, &rp);
            if (rc) return rc;
            dp.fx = rp.fx; dp.fy = rp.fy; dp.x1 = rp.x1; dp.y1 = rp.y1; dp.x2 = rp.x2; dp.y2 = rp.y2;
            if (rp.target_width <= 0 || rp.target_height <= 0) {
                /* A PRESERVE_AR target that rounds to zero columns or rows (a crop more than about
                   2 * dst : 1 off the destination's aspect ratio): the reference's factors become
                   infinite and its region of interest empty (resize.h:127-158), so every output
                   element takes the default value.  The plane is lowered to store-only work; the
                   infinite step is never used. */
                dp.fx = dp.fy = 1.0f; dp.x1 = 0; dp.y1 = 0; dp.x2 = -1; dp.y2 = -1;
            } else {
                step_exp_x[p.sequence] = std::min(step_exp_x[p.sequence], std::ilogb(rp.fx));
                step_exp_y[p.sequence] = std::min(step_exp_y[p.sequence], std::ilogb(rp.fy));
            }
        }

        /* choose the body */
        const uint64_t out_px = (uint64_t)p.dst_width * p.dst_height;
        uint32_t cls = CLASS_GENERIC;
        uint64_t items = 0;
        if (s.resize_mode == FKB_RESIZE_NONE && !is_default && s.dst_format != FKB_DST_F32_PLANAR3 && s.src_format != FKB_SRC_NV12 &&
            s.pre_kind != PRE_GENERAL) {
            const bool src_u8 = s.src_format == FKB_SRC_U8X3, dst_u8 = s.dst_format == FKB_DST_U8X3_PACKED;
            const uintptr_t sa = src_u8 ? 4 : 16, da = dst_u8 ? 4 : 16;
            const uint8_t* src0 = dp.src + (size_t)p.crop_y * p.src_pitch + (size_t)p.crop_x * spx;
            const bool dense = (uint64_t)p.src_pitch == (uint64_t)p.dst_width * spx && (uint64_t)p.dst_pitch == (uint64_t)p.dst_width * dpx &&
                               (uint32_t)p.crop_width == p.src_width;
            const bool rows_ok = (p.src_pitch % sa) == 0 && (p.dst_pitch % da) == 0;
            if (aligned(src0, sa) && aligned(dp.dst, da) && (dense || rows_ok) && !(src_u8 == false && dst_u8)) {
                cls = src_u8 ? (dst_u8 ? CLASS_FLAT_U8_U8 : CLASS_FLAT_U8_F32) : CLASS_FLAT_F32_F32;
                dp.n_segs = dense ? 1 : p.dst_height;
                dp.seg_pixels = dense ? (uint32_t)out_px : p.dst_width;
                if (dense && out_px > 0xFFFFFFFFull) return fail(FKB_ERR_INVALID_ARGUMENT, "plane %d: too many pixels", i);
                const uint32_t item_px = (uint32_t)flat_item_pixels(src_u8);
                items = (uint64_t)dp.n_segs * ((dp.seg_pixels + item_px - 1) / item_px);
            }
        } else if ((s.resize_mode != FKB_RESIZE_NONE || is_default) && (p.dst_width % PX_PER_THREAD) == 0 && aligned(dp.dst, 16) && (p.dst_pitch % 16) == 0 &&
                   s.pre_kind != PRE_GENERAL) {
            if (s.src_format == FKB_SRC_U8X3 && s.dst_format == FKB_DST_F32_PLANAR3 && (p.dst_channel_stride % 16) == 0) cls = CLASS_RESIZE_U8_PLANAR;
            else if (s.src_format == FKB_SRC_U8X3 && s.dst_format == FKB_DST_F32X3_PACKED) cls = CLASS_RESIZE_U8_PACKED;
            else if (s.src_format == FKB_SRC_NV12 && s.dst_format == FKB_DST_F32X3_PACKED) cls = CLASS_RESIZE_NV12_PACKED;
            if (cls != CLASS_GENERIC) {
                const ResizeTiling t = resize_tiling(p.dst_width, p.dst_height, dp.x1, dp.y1, dp.x2, dp.y2, BLOCK_THREADS);
                items = (uint64_t)t.roi_items + t.bg_items;
                dp.roi_items = t.roi_items; dp.tiles_x = t.tiles_x; dp.gw = t.gw; dp.rs = t.rs;
                if (i == 0) { first_groups = t.n_groups; same_groups = true; }
                else if (t.n_groups != first_groups) same_groups = false;
            }
        }
        if (cls == CLASS_GENERIC) {
            items = (out_px + ITEM_PIXELS_GENERIC - 1) / ITEM_PIXELS_GENERIC;
            dp.gw = p.src_width; /* the generic body's border handling needs the image width */
        }
        dp.plane_class = cls;
        if (i == 0) common_class = cls;
        else {
            if (cls != common_class) common_class = CLASS_MIXED;
        }
        img.item_start[i] = (uint32_t)total;
        total += items;
        if (total > 0x7FFFFFFFull) return fail(FKB_ERR_INVALID_ARGUMENT, "plan needs more than 2^31 thread blocks");

        img.output_pixels += out_px;
        const uint64_t crop_px = is_default ? 0 : (uint64_t)p.crop_width * p.crop_height;
        const uint64_t src_bytes = s.src_format == FKB_SRC_NV12 ? crop_px + crop_px / 2 : s.src_format == FKB_SRC_P010 ? 3 * crop_px
                                   : (s.src_format == FKB_SRC_P210 || s.src_format == FKB_SRC_Y210) ? 4 * crop_px
                                   : s.src_format == FKB_SRC_UYVY ? 2 * crop_px : crop_px * spx;
        img.algorithmic_bytes += src_bytes + out_px * (s.dst_format == FKB_DST_F32_PLANAR3 ? 12 : dpx);
    }
    uint32_t common_chain = 0;
    for (int s = 0; s < d->n_sequences; ++s) {
        DevSeq& ds = img.seqs[s];
        const size_t begin = img.ops.size();
        int dev_n_pre = 0;
        const uint32_t chain = lower_ops(d->sequences[s], ds.n_pre, step_exp_x[s], step_exp_y[s], img.ops, dev_n_pre);
        if (s == 0) common_chain = chain;
        else if (chain != common_chain) common_chain = CHAIN_INTERPRET;
        ds.chain = chain_is_compiled(chain) ? chain : CHAIN_INTERPRET;
        ds.ops_begin = (int32_t)begin;
        ds.n_ops = (int32_t)(img.ops.size() - begin);
        ds.n_pre = dev_n_pre - (int32_t)begin;
        img.max_seq_ops = std::max<uint32_t>(img.max_seq_ops, (uint32_t)ds.n_ops);
        for (size_t k = begin; k < img.ops.size(); ++k) {
            img.n_constant_divisions += img.ops[k].opcode == DEV_OP_DIV_BY_CONSTANT;
            img.n_ieee_divisions += img.ops[k].opcode == FKB_OP_DIV;
        }
    }
    img.item_start[d->n_planes] = (uint32_t)total;
    img.total_items = (uint32_t)total;
    /* Planes of one flat class whose sequences differ, some of them compiled chains: the kernel
       that selects per block (first the chain, then the class) runs each plane's compiled chain,
       where the kernel of the class would interpret them all. */
    if ((common_class == CLASS_FLAT_U8_F32 || common_class == CLASS_FLAT_F32_F32 || common_class == CLASS_FLAT_U8_U8) &&
        !chain_is_compiled(common_chain)) {
        bool any_compiled = false;
        for (const DevSeq& ds : img.seqs) any_compiled = any_compiled || ds.chain != CHAIN_INTERPRET;
        if (any_compiled) common_class = CLASS_MIXED;
    }
    img.launch_class = common_class;
    img.chain = (common_class != CLASS_MIXED && common_class != CLASS_GENERIC && chain_is_compiled(common_chain))
                    ? common_chain : CHAIN_INTERPRET;
    /* uchar3 resize plans whose every plane can stage its bands' source rows in shared memory */
    if (common_class == CLASS_RESIZE_U8_PLANAR || common_class == CLASS_RESIZE_U8_PACKED || common_class == CLASS_MIXED) {
        /* In a plan of several classes the same holds for its uchar3 resize planes, if all of them
           can be staged; planes of other classes keep their items.
           A region wider than the columns one block covers (two per thread) is cut into column
           tiles of whole four-pixel groups, each a plane of its own over the same source: its
           destination starts at the tile, its region is the part of the region inside the tile, and
           seg_pixels tells the kernel where in the whole region its first column lies.  The first
           and last tile also take the columns left and right of the region. */
        const std::vector<DevPlane> user_planes = img.planes;
        std::vector<uint32_t> kept_items; /* per lowered plane: its item count if it is not staged, else 0 */
        bool any_resize = false;
        {
            std::vector<DevPlane> cut;
            const uint32_t max_groups = (uint32_t)BLOCK_THREADS * 2u / PX_PER_THREAD;
            for (size_t u = 0; u < user_planes.size(); ++u) {
                const DevPlane& up = user_planes[u];
                if (up.plane_class != CLASS_RESIZE_U8_PLANAR && up.plane_class != CLASS_RESIZE_U8_PACKED) {
                    cut.push_back(up);
                    kept_items.push_back(img.item_start[u + 1] - img.item_start[u]);
                    continue;
                }
                any_resize = true;
                if (region_empty(up)) { /* store-only plane: one "tile", never cut */
                    cut.push_back(up);
                    kept_items.push_back(0);
                    continue;
                }
                const uint32_t px_bytes = up.plane_class == CLASS_RESIZE_U8_PLANAR ? 4u : 12u;
                const uint32_t g_lo = (uint32_t)up.x1 / PX_PER_THREAD;
                const uint32_t n_groups = (uint32_t)up.x2 / PX_PER_THREAD - g_lo + 1;
                const uint32_t n_tiles = (n_groups + max_groups - 1) / max_groups;
                const uint32_t per_tile = (n_groups + n_tiles - 1) / n_tiles;
                for (uint32_t k = 0; k < n_tiles; ++k) {
                    DevPlane dp = up;
                    const uint32_t c0 = k == 0 ? 0u : (g_lo + k * per_tile) * PX_PER_THREAD;
                    const uint32_t c1 = k == n_tiles - 1 ? up.dst_w : (g_lo + (k + 1) * per_tile) * PX_PER_THREAD;
                    const int r0 = std::max(up.x1, (int)c0), r1 = std::min(up.x2, (int)c1 - 1);
                    dp.dst = up.dst + (size_t)c0 * px_bytes;
                    dp.dst_w = c1 - c0;
                    dp.x1 = r0 - (int)c0; dp.x2 = r1 - (int)c0;
                    dp.seg_pixels = (uint32_t)(r0 - up.x1);
                    cut.push_back(dp);
                    kept_items.push_back(0);
                }
            }
            img.planes = std::move(cut);
        }
        /* A batch of narrow regions only (at most 128 columns, 64 threads across) runs blocks of
           128 threads: the same registers hold twice as many blocks per SM, and a batch of small
           planes is bound by how many block start-ups are in flight. */
        uint32_t staged_threads = common_class == CLASS_MIXED ? (uint32_t)BLOCK_THREADS : 128u;
        for (size_t i = 0; i < img.planes.size(); ++i) {
            if (kept_items[i] != 0) continue;
            const DevPlane& dp = img.planes[i];
            if (region_empty(dp)) continue;
            const uint32_t n_groups = (uint32_t)dp.x2 / PX_PER_THREAD - (uint32_t)dp.x1 / PX_PER_THREAD + 1;
            if (n_groups * (PX_PER_THREAD / 2) > 64u) staged_threads = BLOCK_THREADS;
        }
        std::vector<StagedTiling> st(img.planes.size());
        bool all = any_resize;
        uint32_t stage = 0;
        /* A plan with fewer blocks than the GPU has SMs (the README example: five planes of 60 x 60) is cut into
           shorter bands, down to a few hundred pixels each: the launch is then bound by one short block per SM
           instead of by a handful of long ones. */
        for (uint32_t band_pixels = STAGED_BAND_PIXELS;; band_pixels /= 2) {
            uint64_t bands = 0;
            stage = 0;
            for (size_t i = 0; i < img.planes.size() && all; ++i) {
                if (kept_items[i] != 0) { bands += kept_items[i]; continue; }
                st[i] = staged_tiling(img.planes[i], staged_threads, band_pixels);
                all = st[i].ok;
                stage = std::max(stage, st[i].stage_bytes);
                bands += st[i].n_bands;
            }
            if (!all || bands >= SMALL_GRID_BLOCKS || band_pixels <= STAGED_MIN_BAND_PIXELS) break;
        }
        if (!all) img.planes = user_planes; /* the body that reads taps from global memory takes whole planes */
        if (all) {
            img.item_start.assign(img.planes.size() + 1, 0);
            uint64_t t2 = 0;
            for (size_t i = 0; i < img.planes.size(); ++i) {
                DevPlane& dp = img.planes[i];
                if (kept_items[i] != 0) {
                    img.item_start[i] = (uint32_t)t2;
                    t2 += kept_items[i];
                    continue;
                }
                const uint32_t cls = dp.plane_class == CLASS_RESIZE_U8_PLANAR ? CLASS_RESIZE_U8_PLANAR_STAGED : CLASS_RESIZE_U8_PACKED_STAGED;
                const ResizeTiling rt = resize_tiling(dp.dst_w, dp.dst_h, dp.x1, dp.y1, dp.x2, dp.y2, staged_threads);
                const uint64_t outside_groups = (uint64_t)(dp.dst_h - (uint32_t)(dp.y2 - dp.y1 + 1)) * (dp.dst_w / PX_PER_THREAD);
                const bool fold = outside_groups <= STAGED_FOLD_BG_GROUPS && st[i].n_bands != 0;
                dp.n_segs = fold ? 1u : 0u;
                const uint32_t items = st[i].n_bands + (fold ? 0u : rt.bg_items);
                dp.plane_class = cls;
                dp.roi_items = st[i].n_bands; dp.tiles_x = st[i].band_rows; dp.gw = st[i].gw; dp.rs = st[i].rs;
                img.item_start[i] = (uint32_t)t2;
                t2 += items;
            }
            if (t2 > 0x7FFFFFFFull) return fail(FKB_ERR_INVALID_ARGUMENT, "plan needs more than 2^31 thread blocks");
            img.item_start[img.planes.size()] = (uint32_t)t2;
            img.total_items = (uint32_t)t2;
            img.block_threads = staged_threads;
            img.staged_bytes = STAGED_U8_HEADER_BYTES + stage;
            img.early_copies = true;
            img.tiled_copies = build_tensor_maps(img, st, kept_items);
            if (common_class != CLASS_MIXED) img.launch_class = common_class = img.planes[0].plane_class;
        }
    }
    /* NV12 resize plans whose every plane can stage the luma and chroma rows of its band tiles */
    if (common_class == CLASS_RESIZE_NV12_PACKED) {
        std::vector<Nv12Tiling> st(img.planes.size());
        bool all = true;
        uint32_t stage = 0;
        for (size_t i = 0; i < img.planes.size() && all; ++i) {
            st[i] = nv12_staged_tiling(img.planes[i], BLOCK_THREADS);
            all = st[i].ok;
            stage = std::max(stage, st[i].stage_bytes);
        }
        if (all) {
            uint64_t t2 = 0;
            for (size_t i = 0; i < img.planes.size(); ++i) {
                DevPlane& dp = img.planes[i];
                const ResizeTiling rt = resize_tiling(dp.dst_w, dp.dst_h, dp.x1, dp.y1, dp.x2, dp.y2, BLOCK_THREADS);
                const uint32_t items = st[i].n_bands * st[i].tiles_x + rt.bg_items;
                dp.plane_class = CLASS_RESIZE_NV12_PACKED_STAGED;
                dp.roi_items = st[i].n_bands * st[i].tiles_x; dp.tiles_x = st[i].tiles_x; dp.seg_pixels = st[i].band_rows;
                dp.gw = st[i].gw; dp.rs = st[i].rs;
                img.item_start[i] = (uint32_t)t2;
                t2 += items;
            }
            if (t2 > 0x7FFFFFFFull) return fail(FKB_ERR_INVALID_ARGUMENT, "plan needs more than 2^31 thread blocks");
            img.item_start[img.planes.size()] = (uint32_t)t2;
            img.total_items = (uint32_t)t2;
            img.block_threads = BLOCK_THREADS;
            img.staged_bytes = STAGED_HEADER_BYTES + 2 * NV12_MAX_SPAN + stage;
            img.launch_class = common_class = CLASS_RESIZE_NV12_PACKED_STAGED;
#ifndef FKB_CHECK_BOUNDS /* the checked build finds and copies the rows once it knows what the plane allows */
            img.nv12_early = true;
#endif
        }
    }
    /* A plan whose planes all have the same region width can run with exactly as many threads per
       block as its tiling keeps busy. */
    const bool resize_class = common_class == CLASS_RESIZE_U8_PLANAR || common_class == CLASS_RESIZE_U8_PACKED ||
                              common_class == CLASS_RESIZE_NV12_PACKED;
    if (resize_class && same_groups) {
        const DevPlane& p0 = img.planes[0];
        const uint32_t busy = p0.gw * p0.rs;
        const uint32_t threads = (busy + 31) / 32 * 32;
        if (threads < (uint32_t)BLOCK_THREADS) {
            uint64_t t2 = 0;
            for (size_t i = 0; i < img.planes.size(); ++i) {
                DevPlane& dp = img.planes[i];
                const ResizeTiling t = resize_tiling(dp.dst_w, dp.dst_h, dp.x1, dp.y1, dp.x2, dp.y2, threads);
                dp.roi_items = t.roi_items; dp.tiles_x = t.tiles_x; dp.gw = t.gw; dp.rs = t.rs;
                img.item_start[i] = (uint32_t)t2;
                t2 += (uint64_t)t.roi_items + t.bg_items;
            }
            img.item_start[img.planes.size()] = (uint32_t)t2;
            img.total_items = (uint32_t)t2;
            img.block_threads = threads;
        }
    }
    return FKB_OK;
}

/* ------------------------------------------------------------------------------------ */
/* entry points                                                                         */
/* ------------------------------------------------------------------------------------ */
extern "C" FKB_API int fkb_version(void) { return 100; }

extern "C" FKB_API int fkb_debug_bounds_checked(void) {
#ifdef FKB_CHECK_BOUNDS
    return 1;
#else
    return 0;
#endif
}

extern "C" FKB_API const char* fkb_status_string(int status) {
    switch (status) {
        case FKB_OK: return "ok";
        case FKB_ERR_INVALID_ARGUMENT: return "invalid argument";
        case FKB_ERR_UNSUPPORTED: return "unsupported";
        case FKB_ERR_CUDA: return "CUDA error";
        case FKB_ERR_TOO_LARGE: return "too large";
        case FKB_ERR_NO_DEVICE: return "no CUDA device";
        case FKB_ERR_DEVICE_WAIT: return "a device-side wait ran out";
        case FKB_ERR_DEVICE_BOUNDS: return "an access outside an image was refused (bounds-checking build)";
        default: return "unknown status";
    }
}

extern "C" FKB_API const char* fkb_last_error(void) { return g_last_error; }

static int require_device(int* device) {
    int n = 0;
    const cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
        (void)cudaGetLastError();
        return fail(FKB_ERR_NO_DEVICE, "no usable CUDA device (%s); this library has no CPU fallback",
                    e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
    }
    FKB_CUDA(cudaGetDevice(device));
    return FKB_OK;
}

static fkb_plan_info info_of(const HostImage& img) {
    fkb_plan_info info{};
    info.n_planes = (int32_t)img.n_user_planes;
    info.n_sequences = (int32_t)img.seqs.size();
    info.n_launches = 1;
    info.grid_x = img.total_items;
    info.block_x = img.block_threads;
    info.compiled_chain = img.chain != CHAIN_INTERPRET;
    info.output_pixels = img.output_pixels;
    info.algorithmic_bytes = img.algorithmic_bytes;
    info.device_bytes = img.bytes();
    info.n_constant_divisions = img.n_constant_divisions;
    info.n_ieee_divisions = img.n_ieee_divisions;
    return info;
}

extern "C" FKB_API int fkb_plan_validate(const fkb_plan_desc* desc, fkb_plan_info* out_info) {
    HostImage img;
    const int rc = lower(desc, img);
    if (rc) return rc;
    if (out_info) *out_info = info_of(img);
    return FKB_OK;
}

extern "C" FKB_API int fkb_plan_create(const fkb_plan_desc* desc, fkb_plan** out_plan) {
    if (!out_plan) return fail(FKB_ERR_INVALID_ARGUMENT, "fkb_plan_create: out_plan is NULL");
    NvtxRange range("fkb_plan_create");
    *out_plan = nullptr;
    HostImage img;
    int rc = lower(desc, img);
    if (rc) return rc;
    int device = -1;
    rc = require_device(&device);
    if (rc) return rc;

    fkb_plan* plan = new (std::nothrow) fkb_plan();
    if (!plan) return fail(FKB_ERR_INVALID_ARGUMENT, "out of host memory");
    plan->device = device;
    plan->d_bytes = img.bytes();
    std::vector<unsigned char> staging(plan->d_bytes);
    img.serialize(staging.data());
    cudaError_t e = device_alloc(&plan->d_block, plan->d_bytes);
    if (e == cudaSuccess) e = cudaMemcpy(plan->d_block, staging.data(), plan->d_bytes, cudaMemcpyHostToDevice);
    /* A blocking copy from pageable memory returns once the bytes have left `staging`; their last piece may still be on its
       way to the device.  The plan is launched on the caller's stream, which need not wait for the default stream, so the
       table must have landed before this call returns: a kernel that read a table's unfinished end - its last work items,
       its tensor maps - would run on whatever the allocation held before. */
    if (e == cudaSuccess) e = cudaStreamSynchronize(cudaStreamLegacy);
    if (e != cudaSuccess) {
        if (plan->d_block) device_free(plan->d_block);
        delete plan;
        return fail_cuda(e, "plan upload", __LINE__);
    }
    plan->args = img.args_for(static_cast<const unsigned char*>(plan->d_block));
    plan->launch_class = img.launch_class;
    plan->chain = img.chain;
    plan->resize = std::move(img.resize);
    plan->info = info_of(img);
    *out_plan = plan;
    return FKB_OK;
}

extern "C" FKB_API int fkb_plan_launch(const fkb_plan* plan, void* stream) {
    if (!plan) return fail(FKB_ERR_INVALID_ARGUMENT, "fkb_plan_launch: plan is NULL");
    NvtxRange range("fkb_plan_launch");
    int device = -1;
    FKB_CUDA(cudaGetDevice(&device));
    if (device != plan->device)
        return fail(FKB_ERR_INVALID_ARGUMENT, "fkb_plan_launch: the plan lives on device %d but device %d is current", plan->device, device);
    const cudaError_t e = launch_plan_kernel(plan->launch_class, plan->chain, plan->args, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail_cuda(e, "kernel launch", __LINE__);
    return FKB_OK;
}

extern "C" FKB_API int fkb_plan_get_info(const fkb_plan* plan, fkb_plan_info* out) {
    if (!plan || !out) return fail(FKB_ERR_INVALID_ARGUMENT, "fkb_plan_get_info: NULL argument");
    *out = plan->info;
    return FKB_OK;
}

extern "C" FKB_API int fkb_plan_get_resize_params(const fkb_plan* plan, int32_t index, fkb_resize_params* out) {
    if (!plan || !out) return fail(FKB_ERR_INVALID_ARGUMENT, "fkb_plan_get_resize_params: NULL argument");
    if (index < 0 || (size_t)index >= plan->resize.size())
        return fail(FKB_ERR_INVALID_ARGUMENT, "fkb_plan_get_resize_params: plane %d outside [0, %zu)", index, plan->resize.size());
    *out = plan->resize[index];
    return FKB_OK;
}

static int read_status(const uint32_t* d_status, cudaStream_t stream, uint32_t* out) {
    uint32_t st = 0;
    FKB_CUDA(cudaMemcpyAsync(&st, d_status, sizeof st, cudaMemcpyDeviceToHost, stream));
    FKB_CUDA(cudaStreamSynchronize(stream));
    if (out) *out = st;
    if (st != 0) (void)cudaMemsetAsync(const_cast<uint32_t*>(d_status), 0, sizeof st, stream); /* reported once */
    if (st >= STATUS_BOUNDS_SOURCE)
        return fail(FKB_ERR_DEVICE_BOUNDS, "the bounds-checking build refused an access outside %s (status %u); outputs are incomplete",
                    st == STATUS_BOUNDS_SOURCE ? "a source image" : st == STATUS_BOUNDS_DESTINATION ? "a destination image" : "a block's shared memory", st);
    if (st != 0) return fail(FKB_ERR_DEVICE_WAIT, "a thread block gave up waiting for its asynchronous copies (status %u); outputs are incomplete", st);
    return FKB_OK;
}

extern "C" FKB_API int fkb_plan_check(const fkb_plan* plan, void* stream, uint32_t* device_status) {
    if (!plan) return fail(FKB_ERR_INVALID_ARGUMENT, "fkb_plan_check: plan is NULL");
    return read_status(plan->args.status, static_cast<cudaStream_t>(stream), device_status);
}

extern "C" FKB_API int fkb_plan_set_option(fkb_plan* plan, int option, uint32_t value) {
    if (!plan) return fail(FKB_ERR_INVALID_ARGUMENT, "fkb_plan_set_option: plan is NULL");
    switch (option) {
        case FKB_PLAN_WAIT_LIMIT_US:
            if (value == 0 || value > 4000000u) return fail(FKB_ERR_INVALID_ARGUMENT, "fkb_plan_set_option: wait limit %u us outside [1, 4000000]", value);
            plan->args.wait_limit_us = value;
            return FKB_OK;
        case FKB_PLAN_TEST_EXPECT_EXTRA_BYTES:
            if (value % 16 != 0 || value > 1024u) return fail(FKB_ERR_INVALID_ARGUMENT, "fkb_plan_set_option: surplus of %u bytes is not a multiple of 16 up to 1024", value);
            plan->args.test_extra_bytes = value;
            return FKB_OK;
        case FKB_PLAN_TEST_SHRINK_BOUNDS:
            if (value > 64u) return fail(FKB_ERR_INVALID_ARGUMENT, "fkb_plan_set_option: %u rows to hide is more than 64", value);
            plan->args.test_shrink_bounds = value;
            return FKB_OK;
        default:
            return fail(FKB_ERR_INVALID_ARGUMENT, "fkb_plan_set_option: unknown option %d", option);
    }
}

extern "C" FKB_API int fkb_plan_destroy(fkb_plan* plan) {
    if (!plan) return FKB_OK;
    cudaError_t e = cudaSuccess;
    if (plan->d_block) e = device_free(plan->d_block);
    delete plan;
    if (e != cudaSuccess) return fail_cuda(e, "cudaFree", __LINE__);
    return FKB_OK;
}

extern "C" FKB_API int fkb_execute(const fkb_plan_desc* desc, void* stream) {
    fkb_plan* plan = nullptr;
    int rc = fkb_plan_create(desc, &plan);
    if (rc) return rc;
    rc = fkb_plan_launch(plan, stream);
    const cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    int rs = FKB_OK;
    if (rc == FKB_OK && e == cudaSuccess) rs = fkb_plan_check(plan, stream, nullptr);
    fkb_plan_destroy(plan);
    if (rc) return rc;
    if (e != cudaSuccess) return fail_cuda(e, "cudaStreamSynchronize", __LINE__);
    return rs;
}

/* ------------------------------------------------------------------------------------ */
/* asynchronous, allocation-free variant                                                */
/* ------------------------------------------------------------------------------------ */
/* fkb_execute_async is the launch of executors.h:284-285 as this library can make it: lowering on
 * the host, one stream-ordered copy of the descriptor table, the kernel, cudaGetLastError.  Device
 * and pinned memory come from one arena per device that is allocated by the first call and kept
 * until the process ends; tables are placed in it as in a ring, and a table whose range is needed
 * again is released only after the launches that used it have finished (one event per table). */
namespace {

struct AsyncTable {
    size_t off = 0, bytes = 0;          /* range in the arena (0 bytes: a plan that travels in the kernel arguments) */
    cudaEvent_t last_use = nullptr;     /* recorded behind the latest launch that reads the table */
    cudaEvent_t uploaded = nullptr;     /* recorded behind the copy, for launches on another stream */
    cudaStream_t upload_stream = nullptr;
    uint64_t hash = 0;
    std::vector<unsigned char> key;     /* the description, byte for byte */
    LaunchArgs args{};
    uint32_t launch_class = 0, chain = 0;
};

struct AsyncArena {
    std::mutex mu;
    unsigned char* dev = nullptr;       /* | status word (256 B) | ring of FKB_ASYNC_ARENA_BYTES | */
    unsigned char* pinned = nullptr;    /* the ring's staging copy in page-locked host memory */
    size_t head = 0;
    std::deque<AsyncTable> tables;      /* resident tables, oldest first */
    std::vector<cudaEvent_t> spare_events;
};
constexpr size_t ASYNC_HEADER = 256;
constexpr size_t ASYNC_MAX_CACHED = 16; /* descriptions remembered per device */
AsyncArena g_async[64];

cudaError_t arena_event(AsyncArena& ar, cudaEvent_t* ev) {
    if (!ar.spare_events.empty()) { *ev = ar.spare_events.back(); ar.spare_events.pop_back(); return cudaSuccess; }
    return cudaEventCreateWithFlags(ev, cudaEventDisableTiming);
}

/* Releases the oldest table: waits for its launches, keeps its events for reuse. */
cudaError_t arena_release_oldest(AsyncArena& ar) {
    AsyncTable& t = ar.tables.front();
    cudaError_t e = cudaSuccess;
    if (t.last_use) { e = cudaEventSynchronize(t.last_use); ar.spare_events.push_back(t.last_use); }
    if (t.uploaded) ar.spare_events.push_back(t.uploaded);
    ar.tables.pop_front();
    return e;
}

bool ranges_overlap(size_t a, size_t an, size_t b, size_t bn) { return a < b + bn && b < a + an; }

/* The description as one byte string (pointers included: the same chain over other buffers is another plan). */
void description_key(const fkb_plan_desc* d, std::vector<unsigned char>& key) {
    size_t n = 2 * sizeof(int32_t) + (size_t)d->n_planes * sizeof(fkb_plane);
    for (int s = 0; s < d->n_sequences; ++s) n += 22 * sizeof(int32_t) + (size_t)std::max(d->sequences[s].n_ops, 0) * sizeof(fkb_op);
    key.resize(n);
    unsigned char* o = key.data();
    auto put = [&](const void* p, size_t bytes) { std::memcpy(o, p, bytes); o += bytes; };
    put(&d->n_sequences, 4); put(&d->n_planes, 4);
    for (int s = 0; s < d->n_sequences; ++s) {
        const fkb_sequence& q = d->sequences[s];
        put(&q.src_format, 4); put(&q.dst_format, 4); put(&q.resize_mode, 4); put(&q.n_ops, 4); put(&q.n_pre_ops, 4);
        put(q.background, 12);
        put(&q.border_mode, 4); put(q.border_value, 12); put(&q.deinterlace, 4); put(q.transform, 36);
        if (q.n_ops > 0) put(q.ops, (size_t)q.n_ops * sizeof(fkb_op));
    }
    put(d->planes, (size_t)d->n_planes * sizeof(fkb_plane));
}
uint64_t fnv1a(const std::vector<unsigned char>& v) {
    uint64_t h = 1469598103934665603ull;
    const size_t words = v.size() / 8;
    const uint64_t* w = reinterpret_cast<const uint64_t*>(v.data());
    for (size_t i = 0; i < words; ++i) { uint64_t x; std::memcpy(&x, w + i, 8); h = (h ^ x) * 1099511628211ull; }
    for (size_t i = words * 8; i < v.size(); ++i) h = (h ^ v[i]) * 1099511628211ull;
    return h;
}

}  // namespace

extern "C" FKB_API int fkb_execute_async(const fkb_plan_desc* desc, void* stream_) {
    if (!desc || !desc->sequences || !desc->planes || desc->n_sequences <= 0 || desc->n_planes <= 0) {
        HostImage probe;
        return lower(desc, probe); /* reports what is wrong */
    }
    for (int s = 0; s < desc->n_sequences; ++s)
        if (desc->sequences[s].n_ops > 0 && !desc->sequences[s].ops) { HostImage probe; return lower(desc, probe); }
    NvtxRange range("fkb_execute_async");
    int device = -1;
    int rc = require_device(&device);
    if (rc) return rc;
    if (device < 0 || device >= 64) return fail(FKB_ERR_UNSUPPORTED, "fkb_execute_async: device ordinal %d beyond 63", device);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    AsyncArena& ar = g_async[device];
    std::lock_guard<std::mutex> lock(ar.mu);
    if (!ar.dev) { /* first call on this device: the only allocations this entry point ever makes */
        void* d = nullptr; void* h = nullptr;
        cudaError_t e = device_alloc(&d, ASYNC_HEADER + FKB_ASYNC_ARENA_BYTES);
        if (e == cudaSuccess) e = pinned_alloc(&h, FKB_ASYNC_ARENA_BYTES);
        if (e == cudaSuccess) e = cudaMemset(d, 0, ASYNC_HEADER);
        if (e != cudaSuccess) { if (d) device_free(d); if (h) cudaFreeHost(h); return fail_cuda(e, "arena allocation", __LINE__); }
        ar.dev = static_cast<unsigned char*>(d);
        ar.pinned = static_cast<unsigned char*>(h);
    }
    uint32_t* const status = reinterpret_cast<uint32_t*>(ar.dev);

    std::vector<unsigned char> key;
    description_key(desc, key);
    const uint64_t hash = fnv1a(key);
    AsyncTable* t = nullptr;
    for (AsyncTable& c : ar.tables)
        if (c.hash == hash && c.key == key) { t = &c; break; }
    if (t) {
        g_n_reused.fetch_add(1, std::memory_order_relaxed);
        if (t->bytes != 0 && t->upload_stream != stream) FKB_CUDA(cudaStreamWaitEvent(stream, t->uploaded, 0));
    } else {
        HostImage img;
        rc = lower(desc, img);
        if (rc) return rc;
        g_n_lowered.fetch_add(1, std::memory_order_relaxed);
        const bool in_arguments = img.args_for(nullptr).inline_plane != 0;
        const size_t bytes = in_arguments ? 0 : (img.bytes() + 255) & ~(size_t)255;
        if (bytes > FKB_ASYNC_ARENA_BYTES)
            return fail(FKB_ERR_TOO_LARGE, "fkb_execute_async: the plan's descriptor table (%zu bytes) exceeds the arena of %u; use fkb_plan_create", bytes, FKB_ASYNC_ARENA_BYTES);
        while (ar.tables.size() >= ASYNC_MAX_CACHED) FKB_CUDA(arena_release_oldest(ar));
        size_t off = ar.head;
        if (bytes != 0) {
            if (off + bytes > FKB_ASYNC_ARENA_BYTES) off = 0;
            /* tables lie in ring order, so whatever overlaps the new range is at the front */
            for (;;) {
                bool clash = false;
                for (const AsyncTable& c : ar.tables) clash = clash || (c.bytes != 0 && ranges_overlap(off, bytes, c.off, c.bytes));
                if (!clash) break;
                FKB_CUDA(arena_release_oldest(ar));
            }
            ar.head = off + bytes;
        }
        ar.tables.emplace_back();
        t = &ar.tables.back();
        t->off = off; t->bytes = bytes; t->hash = hash; t->key.swap(key);
        t->launch_class = img.launch_class; t->chain = img.chain;
        t->args = img.args_for(ar.dev + ASYNC_HEADER + off);
        t->args.status = status;
        cudaError_t e = arena_event(ar, &t->last_use);
        if (e == cudaSuccess && bytes != 0) e = arena_event(ar, &t->uploaded);
        if (e == cudaSuccess && bytes != 0) {
            img.serialize(ar.pinned + off);
            e = cudaMemcpyAsync(ar.dev + ASYNC_HEADER + off, ar.pinned + off, img.bytes(), cudaMemcpyHostToDevice, stream);
            if (e == cudaSuccess) e = cudaEventRecord(t->uploaded, stream);
            t->upload_stream = stream;
        }
        if (e != cudaSuccess) { ar.tables.pop_back(); return fail_cuda(e, "descriptor upload", __LINE__); }
    }
    const cudaError_t le = launch_plan_kernel(t->launch_class, t->chain, t->args, stream);
    if (le != cudaSuccess) return fail_cuda(le, "kernel launch", __LINE__);
    FKB_CUDA(cudaEventRecord(t->last_use, stream));
    return FKB_OK;
}

extern "C" FKB_API int fkb_async_check(void* stream_, uint32_t* device_status) {
    int device = -1;
    const int rc = require_device(&device);
    if (rc) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (device < 0 || device >= 64 || !g_async[device].dev) { /* nothing was launched here: only the synchronisation */
        FKB_CUDA(cudaStreamSynchronize(stream));
        if (device_status) *device_status = 0;
        return FKB_OK;
    }
    return read_status(reinterpret_cast<uint32_t*>(g_async[device].dev), stream, device_status);
}

/* ------------------------------------------------------------------------------------ */
/* host-buffer variant                                                                  */
/* ------------------------------------------------------------------------------------ */
/* The reference's counterpart is a Ptr allocated as MemType::DeviceAndPinned with
 * upload(stream) before and download(stream) after executeOperations
 * (core/data/ptr_nd.h:252-268,519-530): device mirrors are allocated once and every step
 * copies in, launches and copies out.
 *
 * A session splits the batch by source image: group g holds the planes that read image g and
 * has its own plan.  A step uploads image g, launches group g, and hands the group's outputs
 * to a second stream for the copy back, so that the upload of image g+1 (host to device) runs
 * while the outputs of group g travel the other way. */
struct fkb_host_session {
    struct Copy { void* host; const void* dev; size_t pitch, row_bytes, rows; }; /* rows == 1: plain copy */
    struct Group {
        const void* host_src = nullptr;
        void* dev_src = nullptr;
        size_t src_bytes = 0;
        fkb_plan* plan = nullptr;
        std::vector<Copy> downloads;
        cudaEvent_t computed = nullptr;
    };
    std::vector<Group> groups;
    std::vector<void*> dev_outputs;
    bool external_output = false;      /* the output mirror belongs to the caller (multi-GPU session) */
    cudaStream_t out_stream = nullptr;
    cudaEvent_t start = nullptr, downloaded = nullptr;
    uint64_t h2d_bytes = 0, d2h_bytes = 0;
};

extern "C" FKB_API int fkb_host_session_destroy(fkb_host_session* s) {
    if (!s) return FKB_OK;
    for (auto& g : s->groups) {
        if (g.plan) fkb_plan_destroy(g.plan);
        if (g.dev_src) device_free(g.dev_src);
        if (g.computed) cudaEventDestroy(g.computed);
    }
    if (!s->external_output) for (void* p : s->dev_outputs) if (p) device_free(p);
    if (s->start) cudaEventDestroy(s->start);
    if (s->downloaded) cudaEventDestroy(s->downloaded);
    if (s->out_stream) cudaStreamDestroy(s->out_stream);
    delete s;
    return FKB_OK;
}

/* ext_block != nullptr: the outputs are mirrored inside a device buffer of the caller's in which host address
   ext_lo corresponds to ext_block (the consolidated tensor of a multi-GPU session); the outputs must then tile
   one host range. */
static int host_session_create(const fkb_plan_desc* desc, fkb_host_session** out, unsigned char* ext_block, uintptr_t ext_lo);

extern "C" FKB_API int fkb_host_session_create(const fkb_plan_desc* desc, fkb_host_session** out) {
    return host_session_create(desc, out, nullptr, 0);
}

static int host_session_create(const fkb_plan_desc* desc, fkb_host_session** out, unsigned char* ext_block, uintptr_t ext_lo) {
    if (!out) return fail(FKB_ERR_INVALID_ARGUMENT, "fkb_host_session_create: out is NULL");
    *out = nullptr;
    {
        HostImage probe; /* validates shapes before anything is allocated */
        const int rc = lower(desc, probe);
        if (rc) return rc;
    }
    int device = -1;
    int rc = require_device(&device);
    if (rc) return rc;
    fkb_host_session* s = new (std::nothrow) fkb_host_session();
    if (!s) return fail(FKB_ERR_INVALID_ARGUMENT, "out of host memory");
    auto bail = [&](int code) { fkb_host_session_destroy(s); return code; };

    const int n = desc->n_planes;
    std::vector<fkb_plane> planes(desc->planes, desc->planes + n);

    /* extent of every plane's output in host memory */
    std::vector<size_t> out_bytes(n), out_payload(n);
    uintptr_t lo = UINTPTR_MAX, hi = 0;
    size_t sum = 0;
    for (int i = 0; i < n; ++i) {
        const fkb_plane& p = desc->planes[i];
        const fkb_sequence& q = desc->sequences[p.sequence];
        const size_t row = (size_t)p.dst_width * dst_pixel_bytes(q.dst_format);
        out_bytes[i] = (q.dst_format == FKB_DST_F32_PLANAR3 ? 2 * (size_t)p.dst_channel_stride : 0) +
                       (size_t)p.dst_pitch * (p.dst_height - 1) + row;
        out_payload[i] = (q.dst_format == FKB_DST_F32_PLANAR3 ? 3 : 1) * row * p.dst_height;
        lo = std::min(lo, reinterpret_cast<uintptr_t>(p.dst));
        hi = std::max(hi, reinterpret_cast<uintptr_t>(p.dst) + out_bytes[i]);
        sum += out_payload[i];
    }
    /* Outputs that tile one host range without gaps (a dense tensor) get one device mirror;
       anything else is mirrored and copied plane by plane, row-exact. */
    const bool one_block = (hi - lo) == sum;
    unsigned char* block = nullptr;
    if (ext_block) {
        if (!one_block) return bail(fail(FKB_ERR_UNSUPPORTED, "a consolidated output needs outputs that tile one dense tensor"));
        block = ext_block + (lo - ext_lo);
        s->external_output = true;
    } else if (one_block) {
        void* b = nullptr;
        const cudaError_t e = device_alloc(&b, hi - lo);
        if (e != cudaSuccess) return bail(fail_cuda(e, "output mirror allocation", __LINE__));
        s->dev_outputs.push_back(b);
        block = static_cast<unsigned char*>(b);
    }

    /* groups: planes by source image, in order of first use */
    std::map<const void*, size_t> group_of;
    std::vector<std::vector<int>> members;
    for (int i = 0; i < n; ++i) {
        const fkb_plane& p = desc->planes[i];
        const fkb_sequence& q = desc->sequences[p.sequence];
        const bool is_default = (p.flags & FKB_PLANE_DEFAULT_VALUE) != 0; /* reads no image: a group without an upload */
        const size_t rows = source_rows(q.src_format, p.src_height);
        const size_t bytes = is_default ? 0 : (size_t)p.src_pitch * rows;
        auto it = group_of.find(is_default ? nullptr : p.src);
        if (it == group_of.end()) {
            fkb_host_session::Group g;
            g.host_src = is_default ? nullptr : p.src;
            g.src_bytes = bytes;
            const cudaError_t e = bytes ? device_alloc(&g.dev_src, bytes) : cudaSuccess;
            if (e != cudaSuccess) return bail(fail_cuda(e, "source mirror allocation", __LINE__));
            s->groups.push_back(g);
            members.emplace_back();
            s->h2d_bytes += bytes;
            it = group_of.emplace(is_default ? nullptr : p.src, s->groups.size() - 1).first;
        } else if (s->groups[it->second].src_bytes != bytes) {
            return bail(fail(FKB_ERR_INVALID_ARGUMENT, "plane %d: one source pointer is described with two sizes", i));
        }
        members[it->second].push_back(i);
        planes[i].src = s->groups[it->second].dev_src;
    }

    for (size_t g = 0; g < s->groups.size(); ++g) {
        fkb_host_session::Group& grp = s->groups[g];
        std::vector<fkb_plane> sub;
        for (int i : members[g]) {
            const fkb_plane& p = desc->planes[i];
            const fkb_sequence& q = desc->sequences[p.sequence];
            if (one_block) {
                planes[i].dst = block + (reinterpret_cast<uintptr_t>(p.dst) - lo);
            } else {
                void* mirror = nullptr;
                const cudaError_t e = device_alloc(&mirror, out_bytes[i]);
                if (e != cudaSuccess) return bail(fail_cuda(e, "output mirror allocation", __LINE__));
                s->dev_outputs.push_back(mirror);
                planes[i].dst = mirror;
            }
            sub.push_back(planes[i]);
            const bool dense = out_bytes[i] == out_payload[i]; /* no padding inside this plane's output */
            if (dense) {
                grp.downloads.push_back({p.dst, planes[i].dst, out_bytes[i], out_bytes[i], 1});
            } else {
                const size_t row = (size_t)p.dst_width * dst_pixel_bytes(q.dst_format);
                const int channels = q.dst_format == FKB_DST_F32_PLANAR3 ? 3 : 1;
                for (int c = 0; c < channels; ++c) {
                    const size_t off = (size_t)c * p.dst_channel_stride;
                    grp.downloads.push_back({static_cast<unsigned char*>(p.dst) + off, static_cast<unsigned char*>(planes[i].dst) + off,
                                             p.dst_pitch, row, p.dst_height});
                }
            }
            s->d2h_bytes += out_payload[i];
        }
        /* Outputs of one dense tensor: neighbouring planes merge into runs, and runs of equal size
           at a constant distance (a batch dealt round-robin over the images) come back as one
           strided copy. */
        if (one_block && grp.downloads.size() == members[g].size() && grp.downloads.size() > 1) {
            auto& dl = grp.downloads;
            std::sort(dl.begin(), dl.end(), [](const fkb_host_session::Copy& x, const fkb_host_session::Copy& y) { return x.host < y.host; });
            std::vector<fkb_host_session::Copy> runs;
            for (const auto& d : dl) {
                if (!runs.empty() && d.rows == 1 && runs.back().rows == 1 &&
                    static_cast<unsigned char*>(runs.back().host) + runs.back().row_bytes == d.host) {
                    runs.back().row_bytes += d.row_bytes;
                    runs.back().pitch = runs.back().row_bytes;
                } else {
                    runs.push_back(d);
                }
            }
            bool regular = runs.size() > 1 && runs[0].rows == 1;
            const ptrdiff_t step = regular ? static_cast<unsigned char*>(runs[1].host) - static_cast<unsigned char*>(runs[0].host) : 0;
            for (size_t k = 1; k < runs.size() && regular; ++k)
                regular = runs[k].rows == 1 && runs[k].row_bytes == runs[0].row_bytes &&
                          static_cast<unsigned char*>(runs[k].host) - static_cast<unsigned char*>(runs[0].host) == step * (ptrdiff_t)k;
            if (regular) {
                fkb_host_session::Copy c = runs[0];
                c.pitch = (size_t)step;
                c.rows = runs.size();
                runs.assign(1, c);
            }
            dl.swap(runs);
        }
        fkb_plan_desc dd = *desc;
        dd.planes = sub.data();
        dd.n_planes = (int32_t)sub.size();
        rc = fkb_plan_create(&dd, &grp.plan);
        if (rc) return bail(rc);
        const cudaError_t e = cudaEventCreateWithFlags(&grp.computed, cudaEventDisableTiming);
        if (e != cudaSuccess) return bail(fail_cuda(e, "cudaEventCreate", __LINE__));
    }
    cudaError_t e = cudaStreamCreateWithFlags(&s->out_stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&s->start, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&s->downloaded, cudaEventDisableTiming);
    if (e != cudaSuccess) return bail(fail_cuda(e, "stream / event creation", __LINE__));
    *out = s;
    return FKB_OK;
}

/* Uploads, launches and (if asked) copies back, without synchronising; `stream` ends up behind all of it. */
static int host_session_enqueue(fkb_host_session* s, cudaStream_t stream, bool downloads);

extern "C" FKB_API int fkb_host_session_run(fkb_host_session* s, void* stream_) {
    if (!s) return fail(FKB_ERR_INVALID_ARGUMENT, "fkb_host_session_run: session is NULL");
    NvtxRange range("fkb_host_session_run");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const int rc = host_session_enqueue(s, stream, true);
    if (rc) return rc;
    FKB_CUDA(cudaStreamSynchronize(stream));
    for (auto& g : s->groups) {
        const int rs = fkb_plan_check(g.plan, stream, nullptr);
        if (rs) return rs;
    }
    return FKB_OK;
}

static int host_session_enqueue(fkb_host_session* s, cudaStream_t stream, bool downloads) {
    /* the copy-back stream starts after whatever the caller already queued on `stream` */
    FKB_CUDA(cudaEventRecord(s->start, stream));
    FKB_CUDA(cudaStreamWaitEvent(s->out_stream, s->start, 0));
    for (auto& g : s->groups) {
        if (g.src_bytes) FKB_CUDA(cudaMemcpyAsync(g.dev_src, g.host_src, g.src_bytes, cudaMemcpyHostToDevice, stream));
        const int rc = fkb_plan_launch(g.plan, stream);
        if (rc) return rc;
        if (!downloads) continue;
        FKB_CUDA(cudaEventRecord(g.computed, stream));
        FKB_CUDA(cudaStreamWaitEvent(s->out_stream, g.computed, 0));
        for (const auto& d : g.downloads) {
            if (d.rows == 1) FKB_CUDA(cudaMemcpyAsync(d.host, d.dev, d.row_bytes, cudaMemcpyDeviceToHost, s->out_stream));
            else FKB_CUDA(cudaMemcpy2DAsync(d.host, d.pitch, d.dev, d.pitch, d.row_bytes, d.rows, cudaMemcpyDeviceToHost, s->out_stream));
        }
    }
    FKB_CUDA(cudaEventRecord(s->downloaded, s->out_stream));
    FKB_CUDA(cudaStreamWaitEvent(stream, s->downloaded, 0));
    return FKB_OK;
}

extern "C" FKB_API int fkb_host_session_get_traffic(const fkb_host_session* s, uint64_t* h2d_bytes, uint64_t* d2h_bytes) {
    if (!s || !h2d_bytes || !d2h_bytes) return fail(FKB_ERR_INVALID_ARGUMENT, "fkb_host_session_get_traffic: NULL argument");
    *h2d_bytes = s->h2d_bytes;
    *d2h_bytes = s->d2h_bytes;
    return FKB_OK;
}

extern "C" FKB_API int fkb_execute_host(const fkb_plan_desc* desc, void* stream) {
    fkb_host_session* s = nullptr;
    int rc = fkb_host_session_create(desc, &s);
    if (rc) return rc;
    rc = fkb_host_session_run(s, stream);
    fkb_host_session_destroy(s);
    return rc;
}

/* ------------------------------------------------------------------------------------ */
/* several GPUs of one box                                                              */
/* ------------------------------------------------------------------------------------ */
/* Every output plane depends on its own descriptor and one source image only (the reference indexes
 * opData[thread.z] and nothing else, operation_model/batch_operations.h:153-160), so a batch shards by plane
 * with no exchange step.  The reference's own multi-GPU support ends at a device ordinal on Ptr
 * (core/data/ptr_nd.h:153-165); this session is the dispatcher around it: contiguous plane ranges, one host
 * thread and one stream per device, each device uploads the images its planes read, runs its planes and - on
 * request - copies its outputs back or exchanges them, so that every device holds the consolidated tensor. */

extern "C" FKB_API int fkb_assign_planes(int32_t n_planes, int32_t n_devices, const uint8_t* available, int32_t* first,
                                         int32_t* count) {
    if (n_planes < 0 || n_devices <= 0 || !first || !count)
        return fail(FKB_ERR_INVALID_ARGUMENT, "fkb_assign_planes: bad argument");
    int32_t usable = 0;
    for (int32_t d = 0; d < n_devices; ++d) usable += (!available || available[d]) ? 1 : 0;
    if (usable == 0) return fail(FKB_ERR_NO_DEVICE, "fkb_assign_planes: none of the %d devices is available", n_devices);
    /* contiguous ranges in device order over the devices that answer; sizes differ by at most one plane, so the
       outputs of consecutive devices are consecutive slabs of one tensor */
    const int32_t base = n_planes / usable, extra = n_planes % usable;
    int32_t next = 0, k = 0;
    for (int32_t d = 0; d < n_devices; ++d) {
        if (available && !available[d]) { first[d] = next; count[d] = 0; continue; }
        first[d] = next;
        count[d] = base + (k < extra ? 1 : 0);
        next += count[d];
        ++k;
    }
    return FKB_OK;
}

/* devices a test has declared unavailable (host-side failure injection; no GPU is touched to fake it) */
static std::atomic<uint64_t> g_unavailable_mask{0};
extern "C" FKB_API int fkb_debug_set_device_unavailable(int32_t device, int32_t unavailable) {
    if (device < 0 || device >= 64) return FKB_ERR_INVALID_ARGUMENT;
    if (unavailable) g_unavailable_mask.fetch_or(1ull << device);
    else g_unavailable_mask.fetch_and(~(1ull << device));
    return FKB_OK;
}

namespace {

/* The handful of NCCL entry points the exchange needs, bound at run time so that the library loads where NCCL
   is absent (the exchange is then refused, everything else works). */
struct Nccl {
    typedef struct ncclComm* comm_t;
    int (*CommInitAll)(comm_t*, int, const int*) = nullptr;
    int (*CommDestroy)(comm_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    int (*Broadcast)(const void*, void*, size_t, int /*ncclDataType_t*/, int, comm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    bool ok = false;
};
const Nccl& nccl() {
    static Nccl n;
    static std::once_flag once;
    std::call_once(once, [] {
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) return;
        n.CommInitAll = reinterpret_cast<decltype(n.CommInitAll)>(dlsym(h, "ncclCommInitAll"));
        n.CommDestroy = reinterpret_cast<decltype(n.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
        n.GroupStart = reinterpret_cast<decltype(n.GroupStart)>(dlsym(h, "ncclGroupStart"));
        n.GroupEnd = reinterpret_cast<decltype(n.GroupEnd)>(dlsym(h, "ncclGroupEnd"));
        n.Broadcast = reinterpret_cast<decltype(n.Broadcast)>(dlsym(h, "ncclBroadcast"));
        n.GetErrorString = reinterpret_cast<decltype(n.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
        n.ok = n.CommInitAll && n.CommDestroy && n.GroupStart && n.GroupEnd && n.Broadcast && n.GetErrorString;
    });
    return n;
}

}  // namespace

struct fkb_multi_gpu_session {
    struct Shard {
        int device = -1;
        int32_t first = 0, count = 0;
        fkb_host_session* session = nullptr;
        unsigned char* consolidated = nullptr;  /* FKB_MULTI_GPU_GATHER: the whole output tensor on this device */
        cudaStream_t stream = nullptr;
        cudaEvent_t t0 = nullptr, t1 = nullptr;
        Nccl::comm_t comm = nullptr;
        std::thread worker;
        int rc = FKB_OK;
        std::string error;
        float ms = 0.0f;
    };
    std::vector<Shard> shards;              /* one per device that takes part */
    std::vector<int32_t> requested;         /* the devices as the caller listed them */
    std::vector<int32_t> first, count;      /* per requested device */
    uint32_t flags = 0;
    uintptr_t host_lo = 0;
    size_t out_bytes = 0;
    std::vector<size_t> slab_off, slab_bytes; /* per shard: its slab of the consolidated tensor */
    /* workers wait for `generation` to advance, run one step, and report through `done` */
    std::mutex mu;
    std::condition_variable cv_go, cv_done;
    uint64_t generation = 0;
    int done = 0;
    bool quit = false;
};

static void multi_gpu_step(fkb_multi_gpu_session* m, size_t k) {
    fkb_multi_gpu_session::Shard& sh = m->shards[k];
    NvtxRange range("fkb_multi_gpu_session step");
    auto cuda = [&](cudaError_t e, const char* what) {
        if (e != cudaSuccess && sh.rc == FKB_OK) { sh.rc = FKB_ERR_CUDA; sh.error = std::string(what) + ": " + cudaGetErrorString(e); }
        return e == cudaSuccess;
    };
    sh.rc = FKB_OK;
    sh.error.clear();
    if (!cuda(cudaSetDevice(sh.device), "cudaSetDevice")) return;
    cuda(cudaEventRecord(sh.t0, sh.stream), "cudaEventRecord");
    if (sh.session) {
        const int rc = host_session_enqueue(sh.session, sh.stream, (m->flags & FKB_MULTI_GPU_DOWNLOAD) != 0);
        if (rc) { sh.rc = rc; sh.error = fkb_last_error(); }
    }
    if ((m->flags & FKB_MULTI_GPU_GATHER) && m->shards.size() > 1 && sh.rc == FKB_OK) {
        /* every slab travels from the device that computed it into the same place of every other device's tensor:
           one broadcast per slab, all of them in one group (an all-gather of slabs of unequal size), NCCL moves
           them over NVLink into local memory; no kernel of this library ever reads a peer's memory */
        const Nccl& n = nccl();
        int e = n.GroupStart();
        for (size_t r = 0; r < m->shards.size() && e == 0; ++r)
            if (m->slab_bytes[r]) e = n.Broadcast(sh.consolidated + m->slab_off[r], sh.consolidated + m->slab_off[r], m->slab_bytes[r], 0 /* ncclChar */, (int)r, sh.comm, sh.stream);
        const int e2 = n.GroupEnd();
        if (e == 0) e = e2;
        if (e != 0) { sh.rc = FKB_ERR_CUDA; sh.error = std::string("NCCL: ") + n.GetErrorString(e); }
    }
    cuda(cudaEventRecord(sh.t1, sh.stream), "cudaEventRecord");
    cuda(cudaStreamSynchronize(sh.stream), "cudaStreamSynchronize");
    if (sh.rc == FKB_OK) cuda(cudaEventElapsedTime(&sh.ms, sh.t0, sh.t1), "cudaEventElapsedTime");
    if (sh.rc == FKB_OK && sh.session) {
        for (auto& g : sh.session->groups) {
            const int rc = fkb_plan_check(g.plan, sh.stream, nullptr);
            if (rc) { sh.rc = rc; sh.error = fkb_last_error(); break; }
        }
    }
}

static void multi_gpu_worker(fkb_multi_gpu_session* m, size_t k) {
    uint64_t seen = 0;
    for (;;) {
        {
            std::unique_lock<std::mutex> lock(m->mu);
            m->cv_go.wait(lock, [&] { return m->quit || m->generation != seen; });
            if (m->quit) return;
            seen = m->generation;
        }
        multi_gpu_step(m, k);
        {
            std::lock_guard<std::mutex> lock(m->mu);
            ++m->done;
        }
        m->cv_done.notify_one();
    }
}

extern "C" FKB_API int fkb_multi_gpu_session_destroy(fkb_multi_gpu_session* m) {
    if (!m) return FKB_OK;
    {
        std::lock_guard<std::mutex> lock(m->mu);
        m->quit = true;
    }
    m->cv_go.notify_all();
    for (auto& sh : m->shards) if (sh.worker.joinable()) sh.worker.join();
    for (auto& sh : m->shards) {
        if (cudaSetDevice(sh.device) != cudaSuccess) { (void)cudaGetLastError(); continue; }
        if (sh.comm) nccl().CommDestroy(sh.comm);
        if (sh.session) fkb_host_session_destroy(sh.session);
        if (sh.consolidated) device_free(sh.consolidated);
        if (sh.t0) cudaEventDestroy(sh.t0);
        if (sh.t1) cudaEventDestroy(sh.t1);
        if (sh.stream) cudaStreamDestroy(sh.stream);
    }
    delete m;
    return FKB_OK;
}

extern "C" FKB_API int fkb_multi_gpu_session_create(const fkb_plan_desc* desc, int32_t n_devices, const int32_t* devices, uint32_t flags,
                                                    fkb_multi_gpu_session** out) {
    if (!out) return fail(FKB_ERR_INVALID_ARGUMENT, "fkb_multi_gpu_session_create: out is NULL");
    *out = nullptr;
    if (n_devices <= 0 || n_devices > 64 || !devices) return fail(FKB_ERR_INVALID_ARGUMENT, "fkb_multi_gpu_session_create: between 1 and 64 devices");
    if (flags & ~(uint32_t)(FKB_MULTI_GPU_DOWNLOAD | FKB_MULTI_GPU_GATHER)) return fail(FKB_ERR_INVALID_ARGUMENT, "fkb_multi_gpu_session_create: unknown flag");
    {
        HostImage probe; /* validates the whole description before anything is allocated */
        const int rc = lower(desc, probe);
        if (rc) return rc;
    }
    int present = 0;
    if (cudaGetDeviceCount(&present) != cudaSuccess) { (void)cudaGetLastError(); present = 0; }
    int previous = -1;
    if (present > 0) (void)cudaGetDevice(&previous);
    /* which of the requested devices answer: a device that is missing, that a test declared unavailable, or
       whose context cannot be created is left out and its planes go to the others */
    std::vector<uint8_t> available((size_t)n_devices, 0);
    for (int32_t d = 0; d < n_devices; ++d) {
        const int32_t dev = devices[d];
        if (dev < 0 || dev >= present || dev >= 64) continue;
        if (g_unavailable_mask.load() & (1ull << dev)) continue;
        if (cudaSetDevice(dev) != cudaSuccess || cudaFree(nullptr) != cudaSuccess) { (void)cudaGetLastError(); continue; }
        available[d] = 1;
    }
    fkb_multi_gpu_session* m = new (std::nothrow) fkb_multi_gpu_session();
    if (!m) return fail(FKB_ERR_INVALID_ARGUMENT, "out of host memory");
    m->flags = flags;
    m->requested.assign(devices, devices + n_devices);
    m->first.assign((size_t)n_devices, 0);
    m->count.assign((size_t)n_devices, 0);
    int rc = fkb_assign_planes(desc->n_planes, n_devices, available.data(), m->first.data(), m->count.data());
    auto bail = [&](int code) {
        fkb_multi_gpu_session_destroy(m);
        if (previous >= 0) (void)cudaSetDevice(previous);
        return code;
    };
    if (rc) return bail(rc);

    /* the consolidated tensor: the outputs must tile one host range; a device's slab is the range of its planes */
    uintptr_t lo = UINTPTR_MAX, hi = 0;
    std::vector<uintptr_t> plane_lo((size_t)desc->n_planes), plane_hi((size_t)desc->n_planes);
    for (int i = 0; i < desc->n_planes; ++i) {
        const fkb_plane& p = desc->planes[i];
        const fkb_sequence& q = desc->sequences[p.sequence];
        const size_t row = (size_t)p.dst_width * dst_pixel_bytes(q.dst_format);
        const size_t bytes = (q.dst_format == FKB_DST_F32_PLANAR3 ? 2 * (size_t)p.dst_channel_stride : 0) + (size_t)p.dst_pitch * (p.dst_height - 1) + row;
        plane_lo[i] = reinterpret_cast<uintptr_t>(p.dst);
        plane_hi[i] = plane_lo[i] + bytes;
        lo = std::min(lo, plane_lo[i]);
        hi = std::max(hi, plane_hi[i]);
    }
    m->host_lo = lo;
    m->out_bytes = hi - lo;
    const bool gather = (flags & FKB_MULTI_GPU_GATHER) != 0;
    if (gather && !nccl().ok) return bail(fail(FKB_ERR_UNSUPPORTED, "a consolidated output needs NCCL (libnccl.so.2 was not found)"));

    for (int32_t d = 0; d < n_devices; ++d) {
        if (!available[d]) continue;
        m->shards.emplace_back();
        fkb_multi_gpu_session::Shard& sh = m->shards.back();
        sh.device = devices[d]; sh.first = m->first[d]; sh.count = m->count[d];
    }
    for (auto& sh : m->shards) {
        uintptr_t a = UINTPTR_MAX, b = 0;
        for (int32_t i = sh.first; i < sh.first + sh.count; ++i) { a = std::min(a, plane_lo[i]); b = std::max(b, plane_hi[i]); }
        m->slab_off.push_back(sh.count ? a - lo : 0);
        m->slab_bytes.push_back(sh.count ? b - a : 0);
    }
    for (auto& sh : m->shards) {
        cudaError_t e = cudaSetDevice(sh.device);
        if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&sh.stream, cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaEventCreate(&sh.t0);
        if (e == cudaSuccess) e = cudaEventCreate(&sh.t1);
        if (e == cudaSuccess && gather) {
            void* p = nullptr;
            e = device_alloc(&p, m->out_bytes);
            sh.consolidated = static_cast<unsigned char*>(p);
        }
        if (e != cudaSuccess) return bail(fail_cuda(e, "multi-GPU session set-up", __LINE__));
        if (sh.count > 0) {
            fkb_plan_desc sub = *desc;
            sub.planes = desc->planes + sh.first;
            sub.n_planes = sh.count;
            rc = host_session_create(&sub, &sh.session, sh.consolidated, lo);
            if (rc) return bail(rc);
        }
    }
    if (gather && m->shards.size() > 1) {
        std::vector<Nccl::comm_t> comms(m->shards.size());
        std::vector<int> devs;
        for (auto& sh : m->shards) devs.push_back(sh.device);
        const int e = nccl().CommInitAll(comms.data(), (int)devs.size(), devs.data());
        if (e != 0) return bail(fail(FKB_ERR_CUDA, "ncclCommInitAll: %s", nccl().GetErrorString(e)));
        for (size_t k = 0; k < m->shards.size(); ++k) m->shards[k].comm = comms[k];
    }
    for (size_t k = 0; k < m->shards.size(); ++k) m->shards[k].worker = std::thread(multi_gpu_worker, m, k);
    if (previous >= 0) (void)cudaSetDevice(previous);
    *out = m;
    return FKB_OK;
}

extern "C" FKB_API int fkb_multi_gpu_session_run(fkb_multi_gpu_session* m) {
    if (!m) return fail(FKB_ERR_INVALID_ARGUMENT, "fkb_multi_gpu_session_run: session is NULL");
    {
        std::lock_guard<std::mutex> lock(m->mu);
        m->done = 0;
        ++m->generation;
    }
    m->cv_go.notify_all();
    {
        std::unique_lock<std::mutex> lock(m->mu);
        m->cv_done.wait(lock, [&] { return m->done == (int)m->shards.size(); });
    }
    for (auto& sh : m->shards)
        if (sh.rc != FKB_OK) return fail(sh.rc, "device %d: %s", sh.device, sh.error.c_str());
    return FKB_OK;
}

extern "C" FKB_API int fkb_multi_gpu_session_get_shard(const fkb_multi_gpu_session* m, int32_t index, fkb_multi_gpu_shard* out) {
    if (!m || !out) return fail(FKB_ERR_INVALID_ARGUMENT, "fkb_multi_gpu_session_get_shard: NULL argument");
    if (index < 0 || (size_t)index >= m->requested.size())
        return fail(FKB_ERR_INVALID_ARGUMENT, "fkb_multi_gpu_session_get_shard: device slot %d outside [0, %zu)", index, m->requested.size());
    std::memset(out, 0, sizeof *out);
    out->device = m->requested[(size_t)index];
    out->first_plane = m->first[(size_t)index];
    out->n_planes = m->count[(size_t)index];
    for (const auto& sh : m->shards) {
        if (sh.device != out->device) continue;
        out->available = 1;
        out->consolidated_output = sh.consolidated;
        out->consolidated_bytes = sh.consolidated ? m->out_bytes : 0;
        out->last_step_ms = sh.ms;
    }
    return FKB_OK;
}

/* ------------------------------------------------------------------------------------ */
/* circular tensor                                                                      */
/* ------------------------------------------------------------------------------------ */
struct fkb_circular_tensor {
    fkb_circular_tensor_desc desc{};
    unsigned char* tensor = nullptr;
    unsigned char* ring = nullptr;
    bool own_tensor = false, own_ring = false;
    size_t plane_bytes = 0;
    uint32_t pitch = 0, channel_stride = 0;
    int32_t first = 0;   /* the reference's m_nextUpdateIdx (circular_tensor.h:160) */
    int32_t pos = 0;     /* sliding: first plane of the window */
};

static int check_circular_desc(const fkb_circular_tensor_desc* d) {
    if (!d) return fail(FKB_ERR_INVALID_ARGUMENT, "circular tensor: desc is NULL");
    if (d->width == 0 || d->height == 0 || d->width > 65536 || d->height > 65536)
        return fail(FKB_ERR_INVALID_ARGUMENT, "circular tensor: plane size %ux%u outside [1, 65536]", d->width, d->height);
    if (d->batch < 1 || d->batch > 4096) return fail(FKB_ERR_INVALID_ARGUMENT, "circular tensor: batch %d outside [1, 4096]", d->batch);
    if (d->order != FKB_CIRCULAR_NEWEST_FIRST && d->order != FKB_CIRCULAR_OLDEST_FIRST)
        return fail(FKB_ERR_INVALID_ARGUMENT, "circular tensor: unknown order %d", d->order);
    if (d->dst_format < FKB_DST_F32X3_PACKED || d->dst_format > FKB_DST_U32X3_PACKED)
        return fail(FKB_ERR_INVALID_ARGUMENT, "circular tensor: unknown plane format %d", d->dst_format);
    return FKB_OK;
}

extern "C" FKB_API int fkb_circular_tensor_sizes(const fkb_circular_tensor_desc* d, size_t* plane_bytes, size_t* tensor_bytes,
                                                 size_t* ring_bytes) {
    const int rc = check_circular_desc(d);
    if (rc) return rc;
    const size_t pb = (size_t)d->width * d->height * (d->dst_format == FKB_DST_F32_PLANAR3 ? 12u : dst_pixel_bytes(d->dst_format));
    if (plane_bytes) *plane_bytes = pb;
    if (tensor_bytes) *tensor_bytes = pb * (size_t)d->batch * (d->sliding ? 2 : 1);
    if (ring_bytes) *ring_bytes = d->sliding ? 0 : pb * (size_t)d->batch;
    return FKB_OK;
}

extern "C" FKB_API int fkb_circular_tensor_create(const fkb_circular_tensor_desc* d, fkb_circular_tensor** out) {
    if (!out) return fail(FKB_ERR_INVALID_ARGUMENT, "circular tensor: out is NULL");
    *out = nullptr;
    size_t pb = 0, tb = 0, rb = 0;
    int rc = fkb_circular_tensor_sizes(d, &pb, &tb, &rb);
    if (rc) return rc;
    std::unique_ptr<fkb_circular_tensor> ct(new fkb_circular_tensor());
    ct->desc = *d;
    ct->plane_bytes = pb;
    ct->pitch = d->width * dst_pixel_bytes(d->dst_format);
    ct->channel_stride = d->dst_format == FKB_DST_F32_PLANAR3 ? d->width * d->height * 4u : 0u;
    ct->tensor = static_cast<unsigned char*>(d->tensor);
    ct->ring = d->sliding ? nullptr : static_cast<unsigned char*>(d->ring);
    const bool need_ring = !d->sliding && !ct->ring;
    if (!ct->tensor || need_ring) {
        int device = -1;
        rc = require_device(&device);
        if (rc) return rc;
        void* p = nullptr;
        if (!ct->tensor) {
            FKB_CUDA(device_alloc(&p, tb));
            ct->tensor = static_cast<unsigned char*>(p); ct->own_tensor = true;
            const cudaError_t e = cudaMemset(p, 0, tb);
            if (e != cudaSuccess) { device_free(p); return fail_cuda(e, "cudaMemset", __LINE__); }
        }
        if (need_ring) {
            cudaError_t e = device_alloc(&p, rb);
            if (e == cudaSuccess) { e = cudaMemset(p, 0, rb); if (e != cudaSuccess) device_free(p); }
            if (e != cudaSuccess) { if (ct->own_tensor) device_free(ct->tensor); return fail_cuda(e, "ring allocation", __LINE__); }
            ct->ring = static_cast<unsigned char*>(p); ct->own_ring = true;
        }
    }
    /* the sliding window starts where the first update can move it one plane towards its newest end */
    ct->pos = d->sliding ? (d->order == FKB_CIRCULAR_NEWEST_FIRST ? d->batch : 0) : 0;
    *out = ct.release();
    return FKB_OK;
}

extern "C" FKB_API void* fkb_circular_tensor_data(const fkb_circular_tensor* ct) {
    if (!ct) return nullptr;
    return ct->tensor + (ct->desc.sliding ? (size_t)ct->pos * ct->plane_bytes : 0);
}

extern "C" FKB_API int32_t fkb_circular_tensor_next_index(const fkb_circular_tensor* ct) { return ct ? ct->first : -1; }

extern "C" FKB_API int fkb_circular_tensor_plan_update(fkb_circular_tensor* ct, const fkb_sequence* chain, const fkb_plane* source,
                                                       fkb_sequence* out_sequences, int32_t* n_sequences, fkb_plane* out_planes,
                                                       int32_t* n_planes, int32_t advance) {
    if (!ct || !chain || !source || !out_sequences || !n_sequences || !out_planes || !n_planes)
        return fail(FKB_ERR_INVALID_ARGUMENT, "circular tensor update: NULL argument");
    if (chain->dst_format != ct->desc.dst_format)
        return fail(FKB_ERR_INVALID_ARGUMENT, "circular tensor update: the chain's receiver (format %d) is not the tensor's (%d)",
                    chain->dst_format, ct->desc.dst_format);
    const int32_t B = ct->desc.batch;
    const bool newest_first = ct->desc.order == FKB_CIRCULAR_NEWEST_FIRST;
    auto chain_plane = [&](unsigned char* dst) {
        fkb_plane p = *source;
        p.dst = dst; p.dst_width = ct->desc.width; p.dst_height = ct->desc.height;
        p.dst_pitch = ct->pitch; p.dst_channel_stride = ct->channel_stride; p.sequence = 0;
        return p;
    };
    out_sequences[0] = *chain;
    *n_sequences = 1;
    int32_t n = 0;
    if (ct->desc.sliding) {
        /* window [pos, pos + B) of 2B planes; every result lies at p and p +- B, so the two halves always agree */
        int32_t pos = ct->pos, w;
        if (newest_first) { if (pos == 0) pos = B; pos -= 1; w = pos; }
        else { if (pos == B) pos = 0; pos += 1; w = pos + B - 1; }
        out_planes[n++] = chain_plane(ct->tensor + (size_t)w * ct->plane_bytes);
        out_planes[n++] = chain_plane(ct->tensor + (size_t)(w >= B ? w - B : w + B) * ct->plane_bytes);
        if (advance) ct->pos = pos;
    } else {
        const int32_t first = ct->first;
        const int32_t zu = newest_first ? 0 : B - 1;                  /* SequenceSelectorType (circular_tensor.h:26-35) */
        const int32_t ring_u = (zu + first) % B;                      /* CircularTensorWrite<Ascendent> (memory_operations.h:438-440) */
        /* a copy moves one plane as it lies: whatever the receiver's layout, plane_bytes bytes seen as a packed image */
        fkb_sequence copy{};
        const bool bytes3 = ct->desc.dst_format == FKB_DST_U8X3_PACKED;
        copy.src_format = bytes3 ? FKB_SRC_U8X3 : FKB_SRC_F32X3;
        copy.dst_format = bytes3 ? FKB_DST_U8X3_PACKED : FKB_DST_F32X3_PACKED;
        copy.resize_mode = FKB_RESIZE_NONE;
        const uint32_t copy_pitch = ct->desc.width * (bytes3 ? 3u : 12u);
        for (int32_t z = 0; z < B; ++z) {
            if (z == zu) { out_planes[n++] = chain_plane(ct->tensor + (size_t)z * ct->plane_bytes); continue; }
            int32_t r = newest_first ? first - z : z + first;         /* Descendent / Ascendent (memory_operations.h:437-445) */
            r = r < 0 ? r + B : r >= B ? r - B : r;
            fkb_plane p{};
            p.src = ct->ring + (size_t)r * ct->plane_bytes;
            p.src_width = ct->desc.width; p.src_height = ct->desc.height; p.src_pitch = copy_pitch;
            p.crop_x = 0; p.crop_y = 0; p.crop_width = (int32_t)ct->desc.width; p.crop_height = (int32_t)ct->desc.height;
            p.dst = ct->tensor + (size_t)z * ct->plane_bytes;
            p.dst_width = ct->desc.width; p.dst_height = ct->desc.height; p.dst_pitch = copy_pitch; p.dst_channel_stride = 0;
            p.sequence = 1;
            out_planes[n++] = p;
        }
        out_planes[n++] = chain_plane(ct->ring + (size_t)ring_u * ct->plane_bytes);
        if (B > 1) { out_sequences[1] = copy; *n_sequences = 2; }
        if (advance) ct->first = (first + 1) % B;
    }
    *n_planes = n;
    return FKB_OK;
}

extern "C" FKB_API int fkb_circular_tensor_update(fkb_circular_tensor* ct, const fkb_sequence* chain, const fkb_plane* source, void* stream) {
    if (!ct) return fail(FKB_ERR_INVALID_ARGUMENT, "circular tensor update: NULL tensor");
    NvtxRange range("fkb_circular_tensor_update");
    fkb_sequence seqs[2];
    std::vector<fkb_plane> planes((size_t)ct->desc.batch + 1);
    int32_t ns = 0, np = 0;
    const int32_t first = ct->first, pos = ct->pos;
    int rc = fkb_circular_tensor_plan_update(ct, chain, source, seqs, &ns, planes.data(), &np, 1);
    if (rc) return rc;
    const fkb_plan_desc d{seqs, ns, planes.data(), np};
    rc = fkb_execute_async(&d, stream);
    if (rc) { ct->first = first; ct->pos = pos; } /* nothing ran: the tensor has not moved */
    return rc;
}

extern "C" FKB_API int fkb_circular_tensor_destroy(fkb_circular_tensor* ct) {
    if (!ct) return FKB_OK;
    cudaError_t e = cudaSuccess;
    if (ct->own_tensor) e = device_free(ct->tensor);
    if (ct->own_ring) { const cudaError_t e2 = device_free(ct->ring); if (e == cudaSuccess) e = e2; }
    delete ct;
    if (e != cudaSuccess) return fail_cuda(e, "cudaFree", __LINE__);
    return FKB_OK;
}

/* ------------------------------------------------------------------------------------ */
/* allocation-free variant                                                              */
/* ------------------------------------------------------------------------------------ */
/* fkb_execute_static runs a plan like fkb_execute, but its descriptor table - the only device
 * memory the kernels use beyond the caller's images - lives in the fixed array below instead
 * of a cudaMalloc'ed block.  It is for hosts that must not allocate device memory while they
 * run: a server whose framework reserved the whole of HBM for its own pool at start-up (a
 * cudaMalloc from a plug-in then fails or fragments that pool), and a frame loop with a
 * latency bound, where cudaMalloc and cudaFree stall the host against everything in flight on
 * the device.
 *
 * Every GPU that loads the library holds FKB_STATIC_TABLE_BYTES for this array until the
 * process exits.  All calls on a device share it; it keeps what the last call wrote.  A call
 * rewrites the whole prefix that its kernel reads (planes, sequences, operations, work-item
 * prefix sums) before the launch, in stream order, and the kernel reads nothing beyond that
 * prefix, so nothing has to start at zero. */
static __device__ __align__(256) unsigned char g_static_table[FKB_STATIC_TABLE_BYTES];

/* In host code `g_static_table` is only a handle for the runtime, not a device address; the
 * address on the current device is looked up once per device and cached here. */
static std::mutex g_static_mu;
static unsigned char* g_static_addr[64] = {};

static int static_table_address(int device, unsigned char** out) {
    if (device < 0 || device >= 64) return fail(FKB_ERR_UNSUPPORTED, "fkb_execute_static: device ordinal %d beyond 63", device);
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (!g_static_addr[device]) {
        void* p = nullptr;
        FKB_CUDA(cudaGetSymbolAddress(&p, g_static_table)); /* resolves on the CURRENT device */
        if (!p) return fail(FKB_ERR_CUDA, "fkb_execute_static: the descriptor table has no address on device %d", device);
        g_static_addr[device] = static_cast<unsigned char*>(p);
    }
    *out = g_static_addr[device];
    return FKB_OK;
}

extern "C" FKB_API int fkb_execute_static(const fkb_plan_desc* desc, void* stream_) {
    HostImage img;
    int rc = lower(desc, img);
    if (rc) return rc;
    const size_t bytes = img.bytes();
    if (bytes > (size_t)FKB_STATIC_TABLE_BYTES)
        return fail(FKB_ERR_TOO_LARGE,
                    "fkb_execute_static: the plan needs a descriptor table of %zu bytes (%zu planes, %zu sequences, %zu operations) "
                    "but the fixed table holds %d; split the batch or use fkb_plan_create",
                    bytes, img.planes.size(), img.seqs.size(), img.ops.size(), (int)FKB_STATIC_TABLE_BYTES);
    int device = -1;
    rc = require_device(&device);
    if (rc) return rc;
    unsigned char* table = nullptr;
    rc = static_table_address(device, &table);
    if (rc) return rc;

    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    std::vector<unsigned char> staging(bytes); /* host memory only */
    img.serialize(staging.data());
    /* From pageable memory this returns once `staging` has been read, and is ordered on the
       stream before the launch and after any earlier kernel that still reads the table. */
    FKB_CUDA(cudaMemcpyAsync(table, staging.data(), bytes, cudaMemcpyHostToDevice, stream));
    const LaunchArgs args = img.args_for(table);
    const cudaError_t le = launch_plan_kernel(img.launch_class, img.chain, args, stream);
    /* the status word is read back in stream order, right behind the kernel: a later call on the same
       stream cannot rewrite the table between the kernel and this read */
    uint32_t st = 0;
    const cudaError_t ce = le == cudaSuccess ? cudaMemcpyAsync(&st, args.status, sizeof st, cudaMemcpyDeviceToHost, stream) : cudaSuccess;
    const cudaError_t se = cudaStreamSynchronize(stream);
    if (le != cudaSuccess) return fail_cuda(le, "kernel launch", __LINE__);
    if (ce != cudaSuccess) return fail_cuda(ce, "status read-back", __LINE__);
    if (se != cudaSuccess) return fail_cuda(se, "cudaStreamSynchronize", __LINE__);
    if (st >= STATUS_BOUNDS_SOURCE)
        return fail(FKB_ERR_DEVICE_BOUNDS, "the bounds-checking build refused an access outside %s (status %u); outputs are incomplete",
                    st == STATUS_BOUNDS_SOURCE ? "a source image" : st == STATUS_BOUNDS_DESTINATION ? "a destination image" : "a block's shared memory", st);
    if (st != 0) return fail(FKB_ERR_DEVICE_WAIT, "a thread block gave up waiting for its asynchronous copies (status %u); outputs are incomplete", st);
    return FKB_OK;
}
