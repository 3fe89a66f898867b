/* fkb200 - C ABI of the B200-native fused-execution path.
 *
 * This is the boundary a host front end binds in place of the reference's single launch
 * site: Executor<TransformDPP<ParArch::GPU_NVIDIA,TF>>::executeOperations_helper
 * (core/execution_model/executors.h:252-287), reached from fk::executeOperations
 * (fused_kernel.h:22-54).  The reference passes every instantiable operation by value
 * as a kernel argument (executor_details/executor_kernels.h:25-29) and fixes the batch
 * size at compile time (operation_model/batch_operations.h:98-102); here a sender chain
 * plus its receiver is described by a plain-old-data plan whose batch size is a
 * run-time value and whose per-plane descriptors live in device memory.
 *
 * Conventions: extern "C", plain pointers and sizes, int status return, no exceptions
 * across the boundary, nothing on the device ever traps.  All image pointers inside a
 * plan are DEVICE pointers of the current CUDA device unless a function says otherwise;
 * the library never takes ownership of them (the reference's instantiable operations
 * hold non-owning RawPtr values too, core/data/rawptr.h:124-157).  Launches are
 * asynchronous on the caller's stream, like the reference's (executors.h:284-285).
 */
#ifndef FKB200_H
#define FKB200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define FKB_API __attribute__((visibility("default")))
#else
#define FKB_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------------------ */
/* status codes                                                                         */
/* ------------------------------------------------------------------------------------ */
typedef enum fkb_status {
    FKB_OK = 0,
    FKB_ERR_INVALID_ARGUMENT = 1, /* null pointer, zero size, rect outside its image, ...     */
    FKB_ERR_UNSUPPORTED = 2,      /* a chain shape the kernels do not implement               */
    FKB_ERR_CUDA = 3,             /* a CUDA runtime call failed; see fkb_last_error()         */
    FKB_ERR_TOO_LARGE = 4,        /* beyond a stated capacity (fixed-scratch entry point)     */
    FKB_ERR_NO_DEVICE = 5,        /* no usable CUDA device: there is no CPU fallback          */
    FKB_ERR_DEVICE_WAIT = 6,      /* a kernel gave up a bounded wait; outputs are incomplete  */
    FKB_ERR_DEVICE_BOUNDS = 7     /* bounds-checking build only: a kernel refused an access   */
                                  /* outside its plane's images; outputs are incomplete       */
} fkb_status;

/* ------------------------------------------------------------------------------------ */
/* vocabulary                                                                           */
/* ------------------------------------------------------------------------------------ */

/* Pixel format of a source image (what the chain's read operation returns per element). */
typedef enum fkb_src_format {
    FKB_SRC_U8X3 = 1,  /* PerThreadRead<_2D, uchar3>  (memory_operations.h:71-112)            */
    FKB_SRC_F32X3 = 2, /* PerThreadRead<_2D, float3>                                          */
    FKB_SRC_NV12 = 3,  /* ReadYUV<NV12> (color_conversion.h:314-346): `height` luma rows then */
                       /* height/2 rows of interleaved U,V, chroma at data + pitch*height     */
    FKB_SRC_NV21 = 4,  /* ReadYUV<NV21> (color_conversion.h:347-359): the same with V,U pairs */
    /* The layouts below are read by the one-pixel-per-thread body only, and only as ReadYUV<PF> followed at once by
       ConvertYUVToRGB<PF, Full, ...> (ops[0] is the conversion; its result is float3).  src_width / src_height are
       the image's size in pixels, src_pitch the bytes between rows of its first plane. */
    FKB_SRC_P010 = 5,  /* 4:2:0, 10 bits in the top of 16-bit words: `height` rows of luma words, then height/2    */
                       /* rows of interleaved U,V words at data + pitch*height (color_conversion.h:329-346); the  */
                       /* conversion works on the words shifted right by 6, with chroma offset 512 (luma 64 for    */
                       /* bt601), and multiplies its result by 64 (:284-309, :187-200)                             */
    FKB_SRC_P210 = 6,  /* the same, 4:2:2: `height` rows of chroma                                                 */
    FKB_SRC_Y210 = 7,  /* packed 4:2:2 of 16-bit words Y0 U Y1 V per two pixels (:360-372), 10 bits as above       */
    FKB_SRC_UYVY = 8   /* packed 4:2:2 of bytes U Y0 V Y1 per two pixels (:360-372)                                */
} fkb_src_format;

/* Layout written by the receiver. */
typedef enum fkb_dst_format {
    FKB_DST_F32X3_PACKED = 1, /* PerThreadWrite<_2D,float3> / TensorWrite<float3>             */
                              /* (memory_operations.h:114-137,173-193)                        */
    FKB_DST_F32_PLANAR3 = 2,  /* TensorSplit<float3> (memory_operations.h:195-226): channel c */
                              /* of a plane at byte offset c * channel_stride                 */
    FKB_DST_U8X3_PACKED = 3,  /* PerThreadWrite<_2D,uchar3> / TensorWrite<uchar3>             */
    FKB_DST_I32X3_PACKED = 4, /* PerThreadWrite<_2D,int3> / TensorWrite<int3>: 12 bytes a pixel */
    FKB_DST_U32X3_PACKED = 5  /* PerThreadWrite<_2D,uint3> / TensorWrite<uint3>                 */
} fkb_dst_format;

/* Geometry stage between the read and the element-wise continuation. */
typedef enum fkb_resize_mode {
    FKB_RESIZE_NONE = 0,        /* output element (x,y) reads source element (x,y) of the crop */
    FKB_RESIZE_IGNORE_AR = 1,   /* Resize<INTER_LINEAR, IGNORE_AR>   (resize.h:105-119)         */
    FKB_RESIZE_PRESERVE_AR = 2, /* Resize<INTER_LINEAR, PRESERVE_AR> (resize.h:121-166)         */
    FKB_RESIZE_PRESERVE_AR_RN_EVEN = 3, /* PRESERVE_AR_RN_EVEN: target width (or, when the width is    */
                                /* the limit, height) rounded down to an even number (resize.h:200-210) */
    FKB_RESIZE_PRESERVE_AR_LEFT = 4, /* PRESERVE_AR_LEFT: the region starts at column 0 (resize.h:132-147) */
    FKB_GEOMETRY_WARP_AFFINE = 5,   /* Warping<WarpType::Affine> (image_processing/warping.h:43-104): output (x,y)   */
                                /* reads the source at (m00 x + m01 y + m02, m10 x + m11 y + m12), bilinear like   */
                                /* the resize, 0 where that point lies outside the source                          */
    FKB_GEOMETRY_WARP_PERSPECTIVE = 6 /* Warping<WarpType::Perspective>: the same through a 3x3 matrix (:55-61)   */
} fkb_resize_mode;

/* How the read operation answers coordinates outside its image: BorderReader<BT, Read> (border_reader.h:136-279).
 * With a border mode the crop rect may reach beyond the image (a padded crop): the read chain is
 * PerThreadRead -> BorderReader -> Crop -> geometry stage. */
typedef enum fkb_border_mode {
    FKB_BORDER_NONE = 0,        /* no BorderReader: the crop must lie inside the image                 */
    FKB_BORDER_CONSTANT = 1,    /* `iiiiii|abcdefgh|iiiiiii` with border_value                          */
    FKB_BORDER_REPLICATE = 2,   /* `aaaaaa|abcdefgh|hhhhhhh`                                            */
    FKB_BORDER_REFLECT = 3,     /* `fedcba|abcdefgh|hgfedcb`                                            */
    FKB_BORDER_WRAP = 4,        /* `cdefgh|abcdefgh|abcdefg`                                            */
    FKB_BORDER_REFLECT_101 = 5  /* `gfedcb|abcdefgh|gfedcba`                                            */
} fkb_border_mode;

/* Deinterlace<DType, Read> (deinterlace.h:41-132) between the read and the crop, in image rows. */
typedef enum fkb_deinterlace_mode {
    FKB_DEINTERLACE_NONE = 0,
    FKB_DEINTERLACE_BLEND = 1,        /* (row + row above + 1) * 0.5, the first row as it is (:91-103)   */
    FKB_DEINTERLACE_LINEAR_EVEN = 2,  /* INTER_LINEAR keeping the even rows: odd rows but the last are   */
                                      /* (above + below + 1) * 0.5 (:105-131)                            */
    FKB_DEINTERLACE_LINEAR_ODD = 3    /* keeping the odd rows: even rows but the first are interpolated  */
} fkb_deinterlace_mode;

/* Element-wise operations, applied per channel in IEEE-754 binary32 with no contraction.   */
typedef enum fkb_opcode {
    FKB_OP_MUL = 1,             /* Mul<float3>  v * p   (basic_ops/arithmetic.h:64-75)          */
    FKB_OP_SUB = 2,             /* Sub<float3>  v - p   (arithmetic.h:52-62)                    */
    FKB_OP_DIV = 3,             /* Div<float3>  v / p, true division (arithmetic.h:77-88)       */
    FKB_OP_ADD = 4,             /* Add<float3>  v + p   (arithmetic.h:26-35)                    */
    FKB_OP_CAST_F32 = 5,        /* Cast<uchar3,float3> (basic_ops/cast.h:23-33); exact          */
    FKB_OP_SWAP_RB = 6,         /* ColorConversion<COLOR_RGB2BGR|COLOR_BGR2RGB> =               */
                                /* VectorReorder<T,2,1,0> (basic_ops/cuda_vector.h:50-62)       */
    FKB_OP_SATURATE_CAST_U8 = 7,/* SaturateCast<float3,uchar3> (image_processing/saturate.h)    */
    FKB_OP_YUV_TO_RGB_BT709_FULL = 8, /* ConvertYUVToRGB<NV12,Full,bt709,false,float3>          */
                                /* (color_conversion.h:250-309, matrix :143-146)                */
    FKB_OP_CAST_I32 = 9,        /* Cast<float3,int3>: per-channel static_cast, truncation toward  */
                                /* zero (basic_ops/cast_base.h:20-30, cast.h:23-33).  Last        */
                                /* operation of a sequence only; the receiver is an I32X3 format. */
    FKB_OP_YUV_TO_RGB_BT601_FULL = 11, /* ConvertYUVToRGB<PF,Full,bt601,false,float3>: (Y-16, U-128, V-128) */
                                /* times the matrix of color_conversion.h:137-140 (:266-269)    */
    FKB_OP_YUV_TO_RGB_BT2020_FULL = 12, /* ConvertYUVToRGB<PF,Full,bt2020,false,float3> (:165-168) */
    FKB_OP_CAST_U32 = 10        /* Cast<float3,uint3> (the ending of the reference's run-time test,*/
                                /* tests/operation/test_instantiable_operations.h:241-264).  C++   */
                                /* leaves static_cast of a negative or too large float undefined;  */
                                /* here such values saturate (cvt.rzi.u32.f32).  U32X3 receiver.   */
} fkb_opcode;

typedef struct fkb_op {
    int32_t opcode; /* fkb_opcode */
    float p[3];     /* per-channel parameter of MUL/SUB/DIV/ADD; ignored by the others */
} fkb_op;

/* One operation sequence = one sender chain closed by one receiver kind.
 * ops[0 .. n_pre_ops) run on every tap BEFORE interpolation (they are part of the resize's
 * back operation, as in Read.then(Cast).then(Resize) or ReadYUV.then(ConvertYUVToRGB).then(Resize));
 * ops[n_pre_ops .. n_ops) run on the interpolated value.  With FKB_RESIZE_NONE the split is
 * irrelevant and all ops run in order. */
typedef struct fkb_sequence {
    int32_t src_format;   /* fkb_src_format */
    int32_t dst_format;   /* fkb_dst_format */
    int32_t resize_mode;  /* fkb_resize_mode */
    int32_t n_ops;
    int32_t n_pre_ops;
    float background[3];  /* PRESERVE_AR default value (resize.h:53, :158); the continuation */
                          /* still applies to it (resize.h:84-86).  Also the value that      */
                          /* planes flagged FKB_PLANE_DEFAULT_VALUE read.                    */
    const fkb_op* ops;    /* HOST pointer, n_ops entries (may be NULL when n_ops == 0)       */
    int32_t border_mode;  /* fkb_border_mode                                                  */
    float border_value[3];/* FKB_BORDER_CONSTANT: the value outside the image (source type)   */
    int32_t deinterlace;  /* fkb_deinterlace_mode; the read then returns float3               */
    float transform[9];   /* FKB_GEOMETRY_WARP_*: the matrix, rows of three (affine: two rows) */
} fkb_sequence;

/* One output plane (the reference's thread.z / blockIdx.z, data_parallel_patterns.h:260). */
typedef struct fkb_plane {
    const void* src;        /* source image of this plane                                     */
    uint32_t src_width;     /* in pixels                                                      */
    uint32_t src_height;
    uint32_t src_pitch;     /* bytes between rows (core/data/rawptr.h:205-207)                */
    int32_t crop_x;         /* Crop rect (image_processing/crop.h:35-38, core/data/rect.h);   */
    int32_t crop_y;         /* the whole image when the chain has no Crop                     */
    int32_t crop_width;
    int32_t crop_height;
    void* dst;              /* first element of this plane's output                           */
    uint32_t dst_width;     /* in pixels                                                      */
    uint32_t dst_height;
    uint32_t dst_pitch;     /* bytes between output rows                                      */
    uint32_t dst_channel_stride; /* FKB_DST_F32_PLANAR3: bytes between channel planes         */
    int32_t sequence;       /* index into fkb_plan_desc.sequences (divergent horizontal fusion,*/
                            /* data_parallel_patterns.h:315-323); 0 for an ordinary batch     */
    int32_t flags;          /* FKB_PLANE_* below; 0 for an ordinary plane                      */
} fkb_plane;

/* A plane of a partly filled batch (BatchRead<B, CONDITIONAL_WITH_DEFAULT>, batch_operations.h:217-241:
 * planes at or beyond usedPlanes read `default_value` instead of their image): every element of the read
 * stage is the sequence's `background`, the operations after the geometry stage still apply to it, and
 * the source image is never touched (src may be NULL; the crop is ignored). */
#define FKB_PLANE_DEFAULT_VALUE 1

typedef struct fkb_plan_desc {
    const fkb_sequence* sequences; /* HOST pointer */
    int32_t n_sequences;
    const fkb_plane* planes;       /* HOST pointer */
    int32_t n_planes;
} fkb_plan_desc;

/* Host-derived resize parameters of one plane (Resize::build, resize.h:105-166,196-221). */
typedef struct fkb_resize_params {
    float fx, fy;                    /* source step per output element                         */
    int32_t x1, y1, x2, y2;          /* inclusive region of interest inside the output         */
    int32_t target_width, target_height;
} fkb_resize_params;

/* What a plan will do when launched. */
typedef struct fkb_plan_info {
    int32_t n_planes;
    int32_t n_sequences;
    int32_t n_launches;          /* kernels launched by one fkb_plan_launch                    */
    uint32_t grid_x;             /* grid of the (first) launch                                 */
    uint32_t block_x;
    uint64_t output_pixels;
    uint64_t algorithmic_bytes;  /* source bytes inside the crop rects + output bytes          */
    uint64_t device_bytes;       /* device memory held by the plan's descriptors               */
    int32_t n_constant_divisions;/* Div operations lowered to the proven reciprocal form       */
    int32_t n_ieee_divisions;    /* Div operations kept as IEEE division                       */
    int32_t compiled_chain;      /* 1: the continuation is one of the chains compiled into the  */
                                 /* kernels; 0: it is interpreted from the operation table      */
    int32_t reserved;
} fkb_plan_info;

typedef struct fkb_plan fkb_plan; /* opaque; owns only its own descriptor memory */

/* ------------------------------------------------------------------------------------ */
/* entry points                                                                         */
/* ------------------------------------------------------------------------------------ */

/* Library version, major*10000 + minor*100 + patch. */
FKB_API int fkb_version(void);

/* Human-readable name of a status code. Never NULL. */
FKB_API const char* fkb_status_string(int status);

/* Message of the last failure on the calling thread (empty string if none). */
FKB_API const char* fkb_last_error(void);

/* Restates Resize::build's host arithmetic (resize.h:105-166) and compute_target_size
 * (resize.h:196-221): float scale, cxp::round (constexpr_cmath.h:119-130), double
 * reciprocal narrowed once.  mode is any fkb_resize_mode but FKB_RESIZE_NONE. */
FKB_API int fkb_derive_resize(int32_t src_width, int32_t src_height, int32_t dst_width, int32_t dst_height,
                      int32_t mode, fkb_resize_params* out);

/* Restates the reference's block-shape search getDefaultBlockSize (executors.h:176-242).
 * The kernels here do not use it; it is kept so that a front end can report the grid the
 * reference would have launched. */
FKB_API int fkb_reference_block_size(uint32_t active_x, uint32_t active_y, uint32_t* block_x, uint32_t* block_y);

/* Validates a plan description, derives the per-plane resize parameters and copies the
 * descriptors to the current device.  Replaces the work the reference does at compile
 * time in Fuser::fuseAllIOps (operation_model/iop_fuser.h:44-129) and on the host in
 * BatchRead::build (batch_operations.h:178-208).  The description and everything it
 * points to may be released as soon as the call returns; image memory must stay valid
 * until the launches that use it have finished. */
FKB_API int fkb_plan_create(const fkb_plan_desc* desc, fkb_plan** out_plan);

/* The host half of fkb_plan_create alone: validates and lowers a description and reports what
 * the plan would launch, without touching a device (pointers are checked for NULL and
 * alignment only, never dereferenced). */
FKB_API int fkb_plan_validate(const fkb_plan_desc* desc, fkb_plan_info* out_info);

/* Replaces launchTransformDPP_Kernel<<<grid, block, 0, stream>>> (executors.h:267,270,284)
 * and, for plans with more than one sequence, launchDivergentBatchTransformDPP_Kernel
 * (executor_kernels.h:20-23).  `stream` is a cudaStream_t (NULL = default stream).
 * Asynchronous; returns the launch status only, like the reference's cudaGetLastError check. */
FKB_API int fkb_plan_launch(const fkb_plan* plan, void* stream);

FKB_API int fkb_plan_get_info(const fkb_plan* plan, fkb_plan_info* out_info);

/* Copies the derived resize parameters of plane `index` out of a plan (for parity checks). */
FKB_API int fkb_plan_get_resize_params(const fkb_plan* plan, int32_t index, fkb_resize_params* out);

/* Reads the plan's device status word after synchronising `stream` (the stream of the last
 * launch).  Kernels never trap and never wait without a limit: a thread block whose wait for an
 * asynchronous copy ran out records it there and returns.  *device_status is 0 when every block
 * completed; the call then returns FKB_OK, otherwise FKB_ERR_DEVICE_WAIT and the word is cleared
 * (in stream order), so that one incomplete launch is reported once and later launches of the
 * plan are judged on their own.  The reference has no counterpart (its kernel has no waits); its
 * launch-site check is cudaGetLastError alone (executors.h:285), which fkb_plan_launch keeps. */
FKB_API int fkb_plan_check(const fkb_plan* plan, void* stream, uint32_t* device_status);

/* 1 when this library is the bounds-checking build (libfkb200_check.so: the same sources compiled with
 * -DFKB_CHECK_BOUNDS, every access of a kernel to a source image, a destination or shared memory compared with what
 * the block's plane allows before it is made; an access outside is skipped and reported through the status word as
 * FKB_ERR_DEVICE_BOUNDS, never a fault).  It stands in for a memory checker where none can be run; several times
 * slower, for tests only.  0 in the ordinary build. */
FKB_API int fkb_debug_bounds_checked(void);

/* Run-time options of a plan (fkb_plan_set_option). */
typedef enum fkb_plan_option {
    FKB_PLAN_WAIT_LIMIT_US = 1,       /* longest a thread block waits for its asynchronous copies before it   */
                                      /* records FKB_ERR_DEVICE_WAIT and returns; wall-clock microseconds of  */
                                      /* the GPU's global timer, 1 .. 4,000,000; default FKB_DEFAULT_WAIT_LIMIT_US. */
                                      /* A block that gives up waits once more, as long, for copies still in   */
                                      /* flight towards its shared memory, so it holds an SM for at most twice */
                                      /* the limit.                                                            */
    FKB_PLAN_TEST_EXPECT_EXTRA_BYTES = 2,/* TEST ONLY: every block expects this many bytes more than its copies */
                                      /* deliver (a multiple of 16), so that its wait runs out although every  */
                                      /* copy completed; exercises the give-up path without a fault or a hang. */
    FKB_PLAN_TEST_SHRINK_BOUNDS = 3   /* TEST ONLY, bounds-checking build: the checker treats the last `value`   */
                                      /* rows of every destination as outside, refuses the stores into them and */
                                      /* reports FKB_ERR_DEVICE_BOUNDS; no access outside an image is ever made. */
                                      /* Ignored by the ordinary build.                                         */
} fkb_plan_option;
#define FKB_DEFAULT_WAIT_LIMIT_US 100000u
FKB_API int fkb_plan_set_option(fkb_plan* plan, int option, uint32_t value);

/* Frees the plan's descriptor memory.  Call after the launches that use it have finished. */
FKB_API int fkb_plan_destroy(fkb_plan* plan);

/* One-shot equivalent of fk::executeOperations(stream, sender, receiver) followed by
 * stream.sync(): create, launch, synchronise the stream, destroy. */
FKB_API int fkb_execute(const fkb_plan_desc* desc, void* stream);

/* Asynchronous, allocation-free form of fk::executeOperations(stream, sender, receiver)
 * (fused_kernel.h:22-54 -> executors.h:252-287: one launch, cudaGetLastError, nothing else):
 * validates and lowers `desc`, places the descriptor table in a per-device arena that the
 * library allocates once (device ring + pinned host ring, FKB_ASYNC_ARENA_BYTES each, on the
 * first call on a device), copies it with one stream-ordered cudaMemcpyAsync from pinned memory
 * and launches.  Returns after the launch: it does not synchronise, and after the first call on
 * a device it calls neither cudaMalloc nor cudaFree.  A plan of one plane with up to 16
 * operations travels in the kernel arguments and is not copied at all.  A description equal to
 * one of the last few on the same device (same sequences, planes and pointers: a frame loop over
 * fixed buffers) reuses its lowered table, still resident in the arena, without lowering or
 * copying again.  When the ring is full the call waits for the oldest launch that still holds a
 * slot.  A table larger than the arena is refused with FKB_ERR_TOO_LARGE (use fkb_plan_create).
 * `desc` and what it points to may be released when the call returns. */
#define FKB_ASYNC_ARENA_BYTES (8u * 1024u * 1024u)
FKB_API int fkb_execute_async(const fkb_plan_desc* desc, void* stream);

/* Synchronises `stream` and reports whether any fkb_execute_async launch on the current device
 * since the last check gave up a bounded wait (FKB_ERR_DEVICE_WAIT, cleared by the call); the
 * counterpart of stream.sync() after executeOperations. */
FKB_API int fkb_async_check(void* stream, uint32_t* device_status);

/* Counters for tests: device allocations (cudaMalloc, cudaHostAlloc) and frees made by this
 * library in this process, lowerings skipped because a description was found in the cache. */
typedef struct fkb_debug_counters {
    uint64_t device_allocations, device_frees, host_pinned_allocations, plans_lowered, plans_reused;
} fkb_debug_counters;
FKB_API int fkb_debug_get_counters(fkb_debug_counters* out);

/* Host-buffer sessions: for callers whose images live in HOST memory (preferably pinned).
 * Every pointer in desc->planes (src and dst) is a host pointer.  The reference's
 * counterpart is a Ptr of MemType::DeviceAndPinned with upload(stream) before and
 * download(stream) after executeOperations (core/data/ptr_nd.h:252-268,519-530).
 * create: allocates one device mirror per distinct source image and for the outputs.
 * run:    copies every source in, launches the plan, copies every output back and
 *         synchronises the stream; rows of src_pitch / dst_pitch bytes are assumed and
 *         outputs that tile one host range without gaps come back as a single copy.
 * The description may be released after create; the host images must stay valid. */
typedef struct fkb_host_session fkb_host_session;
FKB_API int fkb_host_session_create(const fkb_plan_desc* desc, fkb_host_session** out_session);
FKB_API int fkb_host_session_run(fkb_host_session* session, void* stream);
FKB_API int fkb_host_session_get_traffic(const fkb_host_session* session, uint64_t* h2d_bytes, uint64_t* d2h_bytes);
FKB_API int fkb_host_session_destroy(fkb_host_session* session);

/* Several GPUs of one box.  Planes are independent (the reference indexes opData[thread.z] alone,
 * operation_model/batch_operations.h:153-160), so a batch shards by plane with no exchange on the hot
 * path; the reference itself stops at a device ordinal on Ptr (core/data/ptr_nd.h:153-165).
 *
 * fkb_assign_planes: contiguous plane ranges over the devices whose `available` byte is non-zero (NULL: all
 * of them), sizes differing by at most one; a device that is not available gets count 0 and its planes go
 * to the others.  Pure host arithmetic.
 *
 * A session takes a description with HOST pointers (like fkb_host_session_create) and a list of CUDA device
 * ordinals.  Devices that do not answer when the session is made are left out and the planes are assigned
 * over the rest (FKB_ERR_NO_DEVICE if none is left).  Each device that takes part gets one host thread and
 * one stream; a step uploads the source images its planes read, launches its planes and, by flag,
 *   FKB_MULTI_GPU_DOWNLOAD  copies its outputs back into the host buffers of the description,
 *   FKB_MULTI_GPU_GATHER    exchanges the output slabs through NCCL (one broadcast per slab, in one group:
 *                           an all-gather of slabs that may differ in size), so that every device holds the
 *                           whole output tensor in its own memory; the outputs must tile one dense host range.
 * run returns when every device has finished its step; times are per device, CUDA events on its stream. */
#define FKB_MULTI_GPU_DOWNLOAD 1u
#define FKB_MULTI_GPU_GATHER 2u
typedef struct fkb_multi_gpu_session fkb_multi_gpu_session;
typedef struct fkb_multi_gpu_shard {
    int32_t device;            /* CUDA ordinal as listed at creation                                   */
    int32_t available;         /* 0: left out (its planes were given to the others)                     */
    int32_t first_plane;       /* the planes of the description this device runs                        */
    int32_t n_planes;
    void* consolidated_output; /* FKB_MULTI_GPU_GATHER: the whole output tensor in this device's memory */
    uint64_t consolidated_bytes;
    float last_step_ms;        /* device time of this device's part of the last run                     */
    int32_t reserved;
} fkb_multi_gpu_shard;
FKB_API int fkb_assign_planes(int32_t n_planes, int32_t n_devices, const uint8_t* available, int32_t* first, int32_t* count);
FKB_API int fkb_multi_gpu_session_create(const fkb_plan_desc* desc, int32_t n_devices, const int32_t* devices, uint32_t flags,
                                         fkb_multi_gpu_session** out_session);
FKB_API int fkb_multi_gpu_session_run(fkb_multi_gpu_session* session);
FKB_API int fkb_multi_gpu_session_get_shard(const fkb_multi_gpu_session* session, int32_t index, fkb_multi_gpu_shard* out);
FKB_API int fkb_multi_gpu_session_destroy(fkb_multi_gpu_session* session);
/* For tests: declares a device ordinal unavailable to sessions made from now on (host-side failure
 * injection; the device itself is not touched). */
FKB_API int fkb_debug_set_device_unavailable(int32_t device, int32_t unavailable);

/* One-shot fkb_host_session_create + run + destroy. */
FKB_API int fkb_execute_host(const fkb_plan_desc* desc, void* stream);

/* ---- a circular tensor: the newest BATCH outputs of a chain, kept in order ----
 * The reference's CircularTensor<T, COLOR_PLANES, BATCH, CT_ORDER, ColorPlanes::Standard>::update
 * (core/data/circular_tensor.h:86-161): every update runs the caller's chain once for one new image and leaves
 * a BATCH-plane tensor whose planes are the last BATCH results, newest first or oldest first, for a
 * model that takes a window of frames.  The reference does it in one divergent launch over BATCH
 * planes (:111-156): one plane runs the chain and stores its result twice - into a hidden ring
 * tensor at plane (z + first) mod BATCH (CircularTensorWrite<Ascendent>, memory_operations.h:436-446,
 * :566-590) and into the visible tensor - and the other BATCH-1 planes copy ring planes into their new
 * visible positions (CircularTensorRead, :531-563: plane z reads ring plane first - z for NewestFirst,
 * z + first for OldestFirst, both mod BATCH); `first` then advances by one (:158).  The plane that
 * runs the chain is 0 for NewestFirst and BATCH-1 for OldestFirst (SequenceSelectorType, :26-35).
 *
 * fkb_circular_tensor_update does the same in one launch of this library's multi-class kernel: a plan of
 * BATCH+1 planes (the chain into the visible plane, the chain into the ring plane, BATCH-1 copies).
 * With `sliding` set the copies disappear: the tensor is a window of BATCH planes inside a buffer
 * of 2*BATCH planes, every result is stored at plane p and p +- BATCH, and the window moves by one plane
 * per update - two stores per update whatever BATCH is, at the price of a data pointer that changes
 * (fkb_circular_tensor_data after every update).  The reference has no such mode.
 * Only the Standard colour-plane mode (plane-major tensors) is built; Transposed needs TensorTSplit
 * windows per channel.  The reference ships no launcher for its divergent kernel (executors.h has
 * no Executor<DivergentBatchTransformDPP>), so update() does not compile there; parity of this
 * entry point is against a restatement of the index arithmetic above. */
typedef enum fkb_circular_order {
    FKB_CIRCULAR_NEWEST_FIRST = 0, /* plane 0 is the latest result */
    FKB_CIRCULAR_OLDEST_FIRST = 1  /* plane BATCH-1 is the latest result */
} fkb_circular_order;

typedef struct fkb_circular_tensor_desc {
    uint32_t width, height; /* of one plane, in pixels                                                   */
    int32_t batch;          /* planes of the visible tensor (1 .. 4096)                                  */
    int32_t order;          /* fkb_circular_order                                                        */
    int32_t dst_format;     /* fkb_dst_format of the planes: the receiver every update's chain ends in   */
    int32_t sliding;        /* 0: the reference's scheme, the tensor stays where it is; 1: sliding window */
    void* tensor;           /* memory for the visible tensor (fkb_circular_tensor_sizes), or NULL to let  */
                            /* the library allocate it on the current device; must hold zeros or earlier  */
                            /* results                                                                   */
    void* ring;             /* memory for the hidden ring, or NULL; unused with `sliding`                 */
} fkb_circular_tensor_desc;

typedef struct fkb_circular_tensor fkb_circular_tensor;

/* Bytes of one plane, of the visible tensor's buffer and of the ring for this description. */
FKB_API int fkb_circular_tensor_sizes(const fkb_circular_tensor_desc* desc, size_t* plane_bytes, size_t* tensor_bytes, size_t* ring_bytes);
/* With both buffers given by the caller nothing is allocated and no CUDA call is made. */
FKB_API int fkb_circular_tensor_create(const fkb_circular_tensor_desc* desc, fkb_circular_tensor** out);
/* First plane of the visible tensor as it is after the latest update; planes are dense (pitch = width * pixel bytes). */
FKB_API void* fkb_circular_tensor_data(const fkb_circular_tensor* ct);
/* The reference's m_nextUpdateIdx (number of updates so far, mod BATCH). */
FKB_API int32_t fkb_circular_tensor_next_index(const fkb_circular_tensor* ct);
/* The plan of the next update, without running it: `chain` is the sender chain and receiver kind of the new image
 * (dst_format must be the tensor's), `source` its plane (source image and crop; destination fields are ignored).
 * out_sequences holds 2 entries, out_planes batch+1.  With `advance` non-zero the tensor moves on as if the plan had
 * run (for callers that run the plan themselves, e.g. together with other planes). */
FKB_API int fkb_circular_tensor_plan_update(fkb_circular_tensor* ct, const fkb_sequence* chain, const fkb_plane* source,
                                            fkb_sequence* out_sequences, int32_t* n_sequences, fkb_plane* out_planes,
                                            int32_t* n_planes, int32_t advance);
/* One update: plans it, runs it with fkb_execute_async on `stream` (asynchronous, no allocation after the
 * library's first call on the device) and advances.  fkb_async_check(stream) waits for it. */
FKB_API int fkb_circular_tensor_update(fkb_circular_tensor* ct, const fkb_sequence* chain, const fkb_plane* source, void* stream);
FKB_API int fkb_circular_tensor_destroy(fkb_circular_tensor* ct);

/* fkb_execute without any device allocation.  No counterpart in the reference (its launch
 * passes all parameters as kernel arguments and never allocates).  Meant for hosts that cannot
 * call cudaMalloc while running: plug-ins inside a server whose framework has taken all of HBM
 * for its own pool, and latency-bound frame loops that cannot afford the device-wide stall of
 * cudaMalloc / cudaFree.  The plan's descriptor table goes into a fixed array of
 * FKB_STATIC_TABLE_BYTES that every GPU loading the library holds until the process exits;
 * image pointers are the caller's, as everywhere else.  Behaviour:
 *  - validates and lowers `desc` exactly like fkb_plan_create, copies the table into the fixed
 *    array on `stream`, launches, and synchronises `stream` before returning;
 *  - a plan whose table (112 B per plane + 128 B per sequence + 16 B per operation + 16 or 32 B
 *    per thread block of its launch) exceeds FKB_STATIC_TABLE_BYTES is refused with
 *    FKB_ERR_TOO_LARGE, nothing runs;
 *  - calls cudaMalloc, cudaFree or an allocating library routine never; host memory only;
 *  - the first call on a device looks up the array's device address (with that device
 *    current), which is also when the CUDA runtime loads this library's module on that device
 *    and reserves the array there; make that first call before the embedding framework takes
 *    the rest of HBM and before starting any stream capture on the device;
 *  - all calls on one device share the array: serialise them per device, whatever their
 *    streams and host threads (two calls that overlap on the GPU race on the array, and two
 *    host threads on one stream would overwrite each other's table before it has been used);
 *  - proving a new Div constant exact costs about 10 ms of host time once per divisor value
 *    and process (see fkb_plan_validate, which can be called at start-up to pay it early). */
#define FKB_STATIC_TABLE_BYTES (512 * 1024)
FKB_API int fkb_execute_static(const fkb_plan_desc* desc, void* stream);

#ifdef __cplusplus
} /* extern "C" */
#endif

#endif /* FKB200_H */
