/* fkb200_executor.h - the reference-side binding of libfkb200: a drop-in at the reference's own
 * extension point.
 *
 * The reference dispatches fk::executeOperations<DPPType>(stream, iops...) (fused_kernel.h:22-54) to
 * fk::Executor<DPPType> (core/execution_model/executors.h:129-145 is the primary template, :245-293
 * the CUDA specialisation whose executeOperations_helper holds the one launch site, :252-287).  This
 * header adds one more data-parallel-pattern tag, fkb200::TransformDPP, and specialises fk::Executor
 * for it: its executeOperations_helper walks the instantiable operations the caller built with the
 * reference's own Op::build(...).then(...) - the values they already carry in OperationData::params /
 * ::backIOp (operation_model/operation_data.h:79-159) - fills a plain-old-data plan and hands it to
 * fkb_execute_async (include/fkb200.h), where the reference would have launched
 * launchTransformDPP_Kernel.  User code changes one template argument:
 *
 *     fk::executeOperations<fk::TransformDPP<>>(stream, sender, receiver);     // the reference's kernel
 *     fk::executeOperations<fkb200::TransformDPP>(stream, sender, receiver);   // this library's kernels
 *
 * All seven overloads of fk::executeOperations work, since they reach the executor through
 * BaseExecutor (executors.h:44-94).  Like the reference's launch it is asynchronous on the stream
 * and allocates nothing (after the library's first call on a device); a chain with an operation
 * outside the path fails to compile with a static_assert naming it, as an unsupported chain does
 * in the reference.  Errors of the library are rethrown as std::runtime_error with the wording of
 * the reference's gpuErrchk (core/utils/utils.h:95-109).
 *
 * Include after <fused_kernel/fused_kernel.h> and <fused_kernel/algorithms/algorithms.h>, in a
 * translation unit compiled by nvcc (the reference defines Stream_<ParArch::GPU_NVIDIA> only there,
 * core/execution_model/stream.h:50).  Needs only include/fkb200.h beside the reference's headers.
 *
 * Operations understood (anything else: static_assert):
 *   reads      PerThreadRead<_2D, uchar3|float3>, ReadYUV<NV12|NV21|P010|P210|Y210|UYVY>, Crop<Back>, Resize<INTER_LINEAR,
 *              IGNORE_AR|PRESERVE_AR|PRESERVE_AR_RN_EVEN|PRESERVE_AR_LEFT, Back>, FusedOperation_<...>,
 *              BatchRead<B, PROCESS_ALL, ...>, BatchRead<B, CONDITIONAL_WITH_DEFAULT, ...>,
 *              BorderReader<BT, Read> directly above the PerThreadRead (a Crop above it may reach beyond the image),
 *              Deinterlace<BLEND|INTER_LINEAR, Read> directly above the PerThreadRead,
 *              Warping<Affine|Perspective, Back> in the place of a Resize
 *   compute    Mul / Sub / Div / Add <float3>, Cast<uchar3,float3>, Cast<float3,int3|uint3>,
 *              SaturateCast<float3,uchar3>, VectorReorder<T,2,1,0> (COLOR_RGB2BGR / COLOR_BGR2RGB),
 *              ConvertYUVToRGB<PF, Full, bt709|bt601|bt2020, false, float3> for the layouts above (directly behind the
 *              read for the four that are not NV12 / NV21)
 *   receivers  PerThreadWrite<_2D|_3D, T>, TensorWrite<T>, TensorSplit<float3>, TensorTSplit<float3>,
 *              SplitWrite<_2D, float3> over three equally spaced images of one pitch
 *
 * The header also supplies the executor the reference declares a pattern for but never defines:
 * fk::Executor<fk::DivergentBatchTransformDPP<ParArch::GPU_NVIDIA, SequenceSelector>> (the pattern:
 * data_parallel_patterns.h:301-353; its only caller: CircularTensor::update, core/data/circular_tensor.h:146).  With this
 * header included, fk::CircularTensor<float, 3, BATCH, order, ColorPlanes::Standard>::update(stream, iops...) compiles
 * and runs as one launch of this library: plane z is lowered from the sequence SequenceSelector::at(z) names, a
 * MidWrite<CircularTensorWrite<...>> directly before the receiver becomes a second store of the plane's result, and
 * CircularTensorRead<dir, TensorRead<T> | TensorPack<float3>, BATCH> becomes BATCH planes that move tensor planes as
 * they lie.  Any other set of sequences closed by receivers works the same way.
 */
#ifndef FKB200_EXECUTOR_H
#define FKB200_EXECUTOR_H

#include <cstring>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <vector>

#include <fkb200.h>

namespace fkb200 {

/* The tag to pass as DPPType.  PAR_ARCH selects the stream type of fk::executeOperations' signature. */
struct TransformDPP {
    static constexpr fk::ParArch PAR_ARCH = fk::ParArch::GPU_NVIDIA;
};

namespace binding {

template <typename T> struct dependent_false : std::false_type {};

/* What is known about one batch plane while its read chain is walked from the outside in. */
struct PlaneState {
    fkb_plane plane{};
    int src_format = 0;
    int resize_mode = FKB_RESIZE_NONE;
    float background[3] = {0.f, 0.f, 0.f};
    std::vector<fkb_op> ops;
    int n_pre_ops = 0;
    bool has_crop = false;
    int border_mode = FKB_BORDER_NONE;
    float border_value[3] = {0.f, 0.f, 0.f};
    int deinterlace = FKB_DEINTERLACE_NONE;
    float transform[9] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    bool raw_planar = false; /* the source is one dense planar float plane (3 x H x W) that is moved as it lies */
    /* what the reference's Resize::build derived on the host (resize.h:105-166), kept so that a caller
       can compare it with what the library derives (fkb_derive_resize) */
    fkb_resize_params reference_resize{};
    bool has_reference_resize = false;
};

inline fkb_op make_op(int opcode, float a = 0.f, float b = 0.f, float c = 0.f) {
    fkb_op o{};
    o.opcode = opcode; o.p[0] = a; o.p[1] = b; o.p[2] = c;
    return o;
}

/* ---- compute operations: LowerCompute<Op>::apply(state[, data]) appends to the plane's operation list ---- */
template <typename Op, typename Enable = void>
struct LowerCompute {
    static_assert(dependent_false<Op>::value, "fkb200: this compute operation is not on the accelerated path");
};
template <typename P> struct LowerCompute<fk::Mul<float3, P, float3>> {
    template <typename D> static void apply(PlaneState& st, const D& d) { st.ops.push_back(make_op(FKB_OP_MUL, d.params.x, d.params.y, d.params.z)); }
};
template <typename P> struct LowerCompute<fk::Sub<float3, P, float3>> {
    template <typename D> static void apply(PlaneState& st, const D& d) { st.ops.push_back(make_op(FKB_OP_SUB, d.params.x, d.params.y, d.params.z)); }
};
template <typename P> struct LowerCompute<fk::Div<float3, P, float3>> {
    template <typename D> static void apply(PlaneState& st, const D& d) { st.ops.push_back(make_op(FKB_OP_DIV, d.params.x, d.params.y, d.params.z)); }
};
template <typename P> struct LowerCompute<fk::Add<float3, P, float3, fk::BinaryType>> {
    template <typename D> static void apply(PlaneState& st, const D& d) { st.ops.push_back(make_op(FKB_OP_ADD, d.params.x, d.params.y, d.params.z)); }
};
template <> struct LowerCompute<fk::Cast<uchar3, float3>> { static void apply(PlaneState& st) { st.ops.push_back(make_op(FKB_OP_CAST_F32)); } };
template <> struct LowerCompute<fk::Cast<float3, int3>> { static void apply(PlaneState& st) { st.ops.push_back(make_op(FKB_OP_CAST_I32)); } };
template <> struct LowerCompute<fk::Cast<float3, uint3>> { static void apply(PlaneState& st) { st.ops.push_back(make_op(FKB_OP_CAST_U32)); } };
template <> struct LowerCompute<fk::SaturateCast<float3, uchar3>> { static void apply(PlaneState& st) { st.ops.push_back(make_op(FKB_OP_SATURATE_CAST_U8)); } };
template <typename T> struct LowerCompute<fk::VectorReorder<T, 2, 1, 0>> { static void apply(PlaneState& st) { st.ops.push_back(make_op(FKB_OP_SWAP_RB)); } };
template <fk::PixelFormat PF> constexpr int yuv_source_format() {
    return PF == fk::PixelFormat::NV12 ? FKB_SRC_NV12 : PF == fk::PixelFormat::NV21 ? FKB_SRC_NV21 : PF == fk::PixelFormat::P010 ? FKB_SRC_P010
           : PF == fk::PixelFormat::P210 ? FKB_SRC_P210 : PF == fk::PixelFormat::Y210 ? FKB_SRC_Y210 : PF == fk::PixelFormat::UYVY ? FKB_SRC_UYVY : 0;
}
template <fk::PixelFormat PF, fk::ColorPrimitives CP> struct LowerCompute<fk::ConvertYUVToRGB<PF, fk::ColorRange::Full, CP, false, float3>> {
    static_assert(yuv_source_format<PF>() != 0, "fkb200: conversions from this pixel format are not on the accelerated path");
    static_assert(CP == fk::ColorPrimitives::bt709 || CP == fk::ColorPrimitives::bt601 || CP == fk::ColorPrimitives::bt2020,
                  "fkb200: this colour matrix is not on the accelerated path");
    static void apply(PlaneState& st) {
        st.ops.push_back(make_op(CP == fk::ColorPrimitives::bt709 ? FKB_OP_YUV_TO_RGB_BT709_FULL
                                 : CP == fk::ColorPrimitives::bt601 ? FKB_OP_YUV_TO_RGB_BT601_FULL : FKB_OP_YUV_TO_RGB_BT2020_FULL));
    }
};

template <typename Op, typename Data>
inline void lower_compute(PlaneState& st, const Data& d) {
    if constexpr (fk::isUnaryType<Op>) LowerCompute<Op>::apply(st);
    else LowerCompute<Op>::apply(st, d);
}

/* ---- read chains ---- */
template <typename Op, typename Enable = void>
struct LowerRead {
    static_assert(dependent_false<Op>::value, "fkb200: this read operation is not on the accelerated path");
};

template <typename T> inline int source_format_of() {
    if constexpr (std::is_same_v<T, uchar3>) return FKB_SRC_U8X3;
    else if constexpr (std::is_same_v<T, float3>) return FKB_SRC_F32X3;
    else { static_assert(dependent_false<T>::value, "fkb200: PerThreadRead of this element type is not on the accelerated path"); return 0; }
}

/* PerThreadRead<_2D, T> (memory_operations.h:71-112): params is the RawPtr of the image */
template <typename T> struct LowerRead<fk::PerThreadRead<fk::ND::_2D, T>> {
    template <typename D> static void apply(PlaneState& st, const D& d) {
        st.src_format = source_format_of<T>();
        st.plane.src = d.params.data;
        st.plane.src_width = d.params.dims.width; st.plane.src_height = d.params.dims.height; st.plane.src_pitch = d.params.dims.pitch;
        st.plane.crop_x = 0; st.plane.crop_y = 0;
        st.plane.crop_width = (int32_t)d.params.dims.width; st.plane.crop_height = (int32_t)d.params.dims.height;
    }
};
/* ReadYUV<NV12> (color_conversion.h:314-400): params is a RawImage whose luma RawPtr has dims.height rows and
   whose chroma plane lies at data + pitch * dims.height (:336-341) */
template <fk::PixelFormat PF> struct LowerRead<fk::ReadYUV<PF>> {
    static_assert(yuv_source_format<PF>() != 0, "fkb200: reads of this pixel format are not on the accelerated path");
    template <typename D> static void apply(PlaneState& st, const D& d) {
        st.src_format = yuv_source_format<PF>();
        st.plane.src = d.params.data.data;
        st.plane.src_width = d.params.width; st.plane.src_height = d.params.data.dims.height; st.plane.src_pitch = d.params.data.dims.pitch;
        st.plane.crop_x = 0; st.plane.crop_y = 0;
        st.plane.crop_width = (int32_t)d.params.width; st.plane.crop_height = (int32_t)d.params.height;
    }
};
/* Crop<Back> (crop.h:23-59): params is the Rect, backIOp the read below it */
template <typename Back> struct LowerRead<fk::Crop<Back>> {
    template <typename D> static void apply(PlaneState& st, const D& d) {
        LowerRead<typename Back::Operation>::apply(st, d.backIOp);
        if (st.resize_mode != FKB_RESIZE_NONE || !st.ops.empty())
            throw std::runtime_error("fkb200: a Crop above a Resize or above compute operations is not on the accelerated path");
        /* crops nest: a rect is relative to the crop below it (crop.h:35-38) */
        st.plane.crop_x += (int32_t)d.params.x; st.plane.crop_y += (int32_t)d.params.y;
        st.plane.crop_width = d.params.width; st.plane.crop_height = d.params.height;
        st.has_crop = true;
    }
};
/* Resize<INTER_LINEAR, AR, Back> (resize.h:61-222): params holds dstSize, the factors and - for PRESERVE_AR - the
   region of interest and the default value that Resize::build computed on the host */
template <fk::AspectRatio AR, typename Back> struct LowerRead<fk::Resize<fk::InterpolationType::INTER_LINEAR, AR, Back>> {

    template <typename D> static void apply(PlaneState& st, const D& d) {
        LowerRead<typename Back::Operation>::apply(st, d.backIOp);
        if (st.resize_mode != FKB_RESIZE_NONE) throw std::runtime_error("fkb200: two Resize operations in one chain are not on the accelerated path");
        st.n_pre_ops = (int)st.ops.size(); /* what the back operation computes runs on every tap, before the interpolation */
        st.plane.dst_width = (uint32_t)d.params.dstSize.width; st.plane.dst_height = (uint32_t)d.params.dstSize.height;
        st.reference_resize.fx = d.params.src_conv_factors.x; st.reference_resize.fy = d.params.src_conv_factors.y;
        st.reference_resize.x1 = 0; st.reference_resize.y1 = 0;
        st.reference_resize.x2 = d.params.dstSize.width - 1; st.reference_resize.y2 = d.params.dstSize.height - 1;
        if constexpr (AR != fk::AspectRatio::IGNORE_AR) {
            st.resize_mode = AR == fk::AspectRatio::PRESERVE_AR ? FKB_RESIZE_PRESERVE_AR
                             : AR == fk::AspectRatio::PRESERVE_AR_RN_EVEN ? FKB_RESIZE_PRESERVE_AR_RN_EVEN : FKB_RESIZE_PRESERVE_AR_LEFT;
            st.background[0] = d.params.defaultValue.x; st.background[1] = d.params.defaultValue.y; st.background[2] = d.params.defaultValue.z;
            st.reference_resize.x1 = d.params.x1; st.reference_resize.y1 = d.params.y1;
            st.reference_resize.x2 = d.params.x2; st.reference_resize.y2 = d.params.y2;
        } else {
            st.resize_mode = FKB_RESIZE_IGNORE_AR;
        }
        st.reference_resize.target_width = st.reference_resize.x2 - st.reference_resize.x1 + 1;
        st.reference_resize.target_height = st.reference_resize.y2 - st.reference_resize.y1 + 1;
        st.has_reference_resize = true;
    }
};

/* BorderReader<BT, Back> (border_reader.h:136-279): params holds the value of a CONSTANT border, backIOp the read whose
   coordinates it folds back into the image.  Only directly above the image read: the library applies the border to
   image coordinates, below the crop. */
template <fk::BorderType BT, typename Back, typename E>
struct LowerRead<fk::BorderReader<BT, Back, E>, std::enable_if_t<!std::is_void_v<Back>>> {
    template <typename D> static void apply(PlaneState& st, const D& d) {
        LowerRead<typename Back::Operation>::apply(st, d.backIOp);
        if (st.has_crop || st.resize_mode != FKB_RESIZE_NONE || !st.ops.empty() || st.border_mode != FKB_BORDER_NONE ||
            st.deinterlace != FKB_DEINTERLACE_NONE)
            throw std::runtime_error("fkb200: a BorderReader anywhere but directly above the image read is not on the accelerated path");
        st.border_mode = BT == fk::BorderType::CONSTANT ? FKB_BORDER_CONSTANT : BT == fk::BorderType::REPLICATE ? FKB_BORDER_REPLICATE
                         : BT == fk::BorderType::REFLECT ? FKB_BORDER_REFLECT : BT == fk::BorderType::WRAP ? FKB_BORDER_WRAP
                         : FKB_BORDER_REFLECT_101;
        if constexpr (BT == fk::BorderType::CONSTANT) {
            st.border_value[0] = (float)d.params.value.x; st.border_value[1] = (float)d.params.value.y; st.border_value[2] = (float)d.params.value.z;
        }
    }
};
/* Deinterlace<DT, Back> (deinterlace.h:41-131): INTER_LINEAR's params say which field is kept; returns float3 */
template <fk::DeinterlaceType DT, typename Back>
struct LowerRead<fk::Deinterlace<DT, Back>, std::enable_if_t<!std::is_void_v<Back>>> {
    template <typename D> static void apply(PlaneState& st, const D& d) {
        LowerRead<typename Back::Operation>::apply(st, d.backIOp);
        if (st.has_crop || st.resize_mode != FKB_RESIZE_NONE || !st.ops.empty() || st.border_mode != FKB_BORDER_NONE ||
            st.deinterlace != FKB_DEINTERLACE_NONE)
            throw std::runtime_error("fkb200: a Deinterlace anywhere but directly above the image read is not on the accelerated path");
        if constexpr (DT == fk::DeinterlaceType::BLEND) st.deinterlace = FKB_DEINTERLACE_BLEND;
        else st.deinterlace = d.params.useEvenLines ? FKB_DEINTERLACE_LINEAR_EVEN : FKB_DEINTERLACE_LINEAR_ODD;
    }
};
/* Warping<WT, Back> (warping.h:43-104): params holds the inverse map (2x3 or 3x3) and the output size */
template <fk::WarpType WT, typename Back>
struct LowerRead<fk::Warping<WT, Back>, std::enable_if_t<!std::is_void_v<Back>>> {
    template <typename D> static void apply(PlaneState& st, const D& d) {
        LowerRead<typename Back::Operation>::apply(st, d.backIOp);
        if (st.resize_mode != FKB_RESIZE_NONE) throw std::runtime_error("fkb200: a Warping above a Resize or another Warping is not on the accelerated path");
        st.n_pre_ops = (int)st.ops.size();
        st.resize_mode = WT == fk::WarpType::Affine ? FKB_GEOMETRY_WARP_AFFINE : FKB_GEOMETRY_WARP_PERSPECTIVE;
        constexpr int rows = WT == fk::WarpType::Affine ? 2 : 3;
        for (int r = 0; r < rows; ++r) for (int c = 0; c < 3; ++c) st.transform[3 * r + c] = d.params.transformMatrix.data[r][c];
        if (rows == 2) { st.transform[6] = 0.f; st.transform[7] = 0.f; st.transform[8] = 1.f; }
        st.plane.dst_width = (uint32_t)d.params.dstSize.width; st.plane.dst_height = (uint32_t)d.params.dstSize.height;
    }
};

/* OperationTuple<Ops...> (operation_tuple.h:22-67): `instance` exists for operations with parameters, `next`
   unless everything from here on is unary, in which case only the types remain */
template <typename Tuple> inline void walk_types_only(PlaneState& st) {
    LowerCompute<typename Tuple::Operation>::apply(st);
    if constexpr (Tuple::size > 1) walk_types_only<typename Tuple::Next>(st);
}
template <typename Tuple> inline void walk_compute_tuple(PlaneState& st, const Tuple& t) {
    using Op = typename Tuple::Operation;
    if constexpr (fk::isUnaryType<Op>) {
        LowerCompute<Op>::apply(st);
        if constexpr (Tuple::size > 1) {
            if constexpr (std::is_empty_v<Tuple>) walk_types_only<typename Tuple::Next>(st);
            else walk_compute_tuple(st, t.next);
        }
    } else {
        LowerCompute<Op>::apply(st, t.instance);
        if constexpr (Tuple::size > 1) walk_compute_tuple(st, t.next);
    }
}
/* FusedOperation_<E, Read, Compute...> (fused_operation.h:136-329): a read followed by the continuation that .then()
   fused onto it; params is the OperationTuple */
template <typename E, typename First, typename... Rest> struct LowerRead<fk::FusedOperation_<E, First, Rest...>, std::enable_if_t<fk::isAnyReadType<First>>> {
    template <typename D> static void apply(PlaneState& st, const D& d) {
        LowerRead<First>::apply(st, d.params.instance);
        if constexpr (sizeof...(Rest) > 0) {
            using Tuple = std::decay_t<decltype(d.params)>;
            if constexpr (std::is_empty_v<typename Tuple::Next>) walk_types_only<typename Tuple::Next>(st);
            else walk_compute_tuple(st, d.params.next);
        }
    }
};
/* a fused continuation handed to executeOperations as one compute operation */
template <typename E, typename First, typename... Rest> struct LowerCompute<fk::FusedOperation_<E, First, Rest...>, std::enable_if_t<fk::isComputeType<First>>> {
    static void apply(PlaneState& st) { walk_types_only<fk::OperationTuple<First, Rest...>>(st); }
    template <typename D> static void apply(PlaneState& st, const D& d) { walk_compute_tuple(st, d.params); }
};

/* ---- receivers ---- */
struct Receiver {
    void* data = nullptr;
    uint32_t width = 0, height = 0, pitch = 0, planes = 1;
    size_t plane_bytes = 0;        /* distance between the outputs of consecutive batch planes */
    uint32_t channel_stride = 0;   /* TensorSplit: bytes between the channel planes of one output */
    int dst_format = 0;
};
template <typename T> inline int packed_format_of() {
    if constexpr (std::is_same_v<T, float3>) return FKB_DST_F32X3_PACKED;
    else if constexpr (std::is_same_v<T, uchar3>) return FKB_DST_U8X3_PACKED;
    else if constexpr (std::is_same_v<T, int3>) return FKB_DST_I32X3_PACKED;
    else if constexpr (std::is_same_v<T, uint3>) return FKB_DST_U32X3_PACKED;
    else { static_assert(dependent_false<T>::value, "fkb200: a receiver of this element type is not on the accelerated path"); return 0; }
}
template <typename Op, typename Enable = void>
struct LowerWrite {
    static_assert(dependent_false<Op>::value, "fkb200: this receiver is not on the accelerated path");
};
template <typename T> struct LowerWrite<fk::PerThreadWrite<fk::ND::_2D, T>> {
    template <typename D> static Receiver apply(const D& d) {
        Receiver r;
        r.data = d.params.data; r.width = d.params.dims.width; r.height = d.params.dims.height; r.pitch = d.params.dims.pitch;
        r.planes = 1; r.plane_bytes = (size_t)r.pitch * r.height; r.dst_format = packed_format_of<T>();
        return r;
    }
};
template <typename D> inline Receiver tensor_receiver(const D& d, int fmt) {
    Receiver r;
    r.data = d.params.data; r.width = d.params.dims.width; r.height = d.params.dims.height; r.pitch = d.params.dims.pitch;
    r.planes = d.params.dims.planes;
    /* plane z starts plane_pitch * color_planes * z bytes in (core/data/rawptr.h:222-225) */
    r.plane_bytes = (size_t)d.params.dims.plane_pitch * d.params.dims.color_planes;
    r.dst_format = fmt;
    return r;
}
template <typename T> struct LowerWrite<fk::PerThreadWrite<fk::ND::_3D, T>> {
    template <typename D> static Receiver apply(const D& d) { return tensor_receiver(d, packed_format_of<T>()); }
};
template <typename T> struct LowerWrite<fk::TensorWrite<T>> {
    template <typename D> static Receiver apply(const D& d) { return tensor_receiver(d, packed_format_of<T>()); }
};
/* TensorSplit<float3> (memory_operations.h:195-226): channel c of a plane lies width*height elements further */
template <> struct LowerWrite<fk::TensorSplit<float3>> {
    template <typename D> static Receiver apply(const D& d) {
        Receiver r = tensor_receiver(d, FKB_DST_F32_PLANAR3);
        r.channel_stride = d.params.dims.width * d.params.dims.height * (uint32_t)sizeof(float);
        return r;
    }
};

/* TensorTSplit<float3> (memory_operations.h:228-255): channel-major over the whole batch, [C][N][H][W]; plane z at
   plane_pitch * z, channel c a further color_planes_pitch * c (core/data/rawptr.h:231-239) */
template <> struct LowerWrite<fk::TensorTSplit<float3>> {
    template <typename D> static Receiver apply(const D& d) {
        Receiver r;
        r.data = d.params.data; r.width = d.params.dims.width; r.height = d.params.dims.height; r.pitch = d.params.dims.pitch;
        r.planes = d.params.dims.planes; r.plane_bytes = d.params.dims.plane_pitch; r.channel_stride = d.params.dims.color_planes_pitch;
        r.dst_format = FKB_DST_F32_PLANAR3;
        return r;
    }
};
/* SplitWrite<_2D, float3> (memory_operations.h:374-407): three images; expressible when they share one pitch and lie at
   equal distances (the planar receiver has one channel stride) */
template <> struct LowerWrite<fk::SplitWrite<fk::ND::_2D, float3>> {
    template <typename D> static Receiver apply(const D& d) {
        const auto& x = d.params.x; const auto& y = d.params.y; const auto& z = d.params.z;
        const ptrdiff_t s1 = reinterpret_cast<const char*>(y.data) - reinterpret_cast<const char*>(x.data);
        const ptrdiff_t s2 = reinterpret_cast<const char*>(z.data) - reinterpret_cast<const char*>(y.data);
        if (s1 <= 0 || s1 != s2 || s1 > 0xFFFFFFFFll || x.dims.pitch != y.dims.pitch || y.dims.pitch != z.dims.pitch)
            throw std::runtime_error("fkb200: SplitWrite needs three images of one pitch at equal, increasing distances below 4 GiB");
        Receiver r;
        r.data = x.data; r.width = x.dims.width; r.height = x.dims.height; r.pitch = x.dims.pitch;
        r.planes = 1; r.plane_bytes = 0; r.channel_stride = (uint32_t)s1; r.dst_format = FKB_DST_F32_PLANAR3;
        return r;
    }
};

/* ---- the whole call ---- */
struct LoweredPlan {
    std::vector<PlaneState> states;
    std::vector<fkb_sequence> sequences;
    std::vector<std::vector<fkb_op>> sequence_ops;
    std::vector<fkb_plane> planes;

    fkb_plan_desc desc() {
        for (size_t s = 0; s < sequences.size(); ++s) sequences[s].ops = sequence_ops[s].empty() ? nullptr : sequence_ops[s].data();
        return fkb_plan_desc{sequences.data(), (int32_t)sequences.size(), planes.data(), (int32_t)planes.size()};
    }
};

/* the first operation: one plane, or BatchRead<B, PROCESS_ALL, Op> (batch_operations.h:135-210) whose params hold
   one OperationData per plane (:98-102) */
template <typename Op> struct LowerFirst {
    template <typename D> static void apply(std::vector<PlaneState>& states, const D& d) {
        states.emplace_back();
        LowerRead<Op>::apply(states.back(), d);
    }
};
template <size_t B, typename Op, typename Out> struct LowerFirst<fk::BatchRead<B, fk::PlanePolicy::PROCESS_ALL, Op, Out>> {
    template <typename D> static void apply(std::vector<PlaneState>& states, const D& d) {
        states.reserve(B);
        for (size_t z = 0; z < B; ++z) {
            states.emplace_back();
            LowerRead<Op>::apply(states.back(), d.params.opData[z]);
        }
    }
};

/* BatchRead<B, CONDITIONAL_WITH_DEFAULT, Op, Out> (batch_operations.h:217-287): planes at or beyond usedPlanes return
   default_value in place of Op's result over the whole active area; operations that follow the batch still apply */
template <size_t B, typename Op, typename Out> struct LowerFirst<fk::BatchRead<B, fk::PlanePolicy::CONDITIONAL_WITH_DEFAULT, Op, Out>> {
    template <typename D> static void apply(std::vector<PlaneState>& states, const D& d) {
        states.reserve(B);
        for (size_t z = 0; z < B; ++z) {
            states.emplace_back();
            PlaneState& st = states.back();
            if ((int)z < d.params.usedPlanes) { LowerRead<Op>::apply(st, d.params.opData[z]); continue; }
            using DV = std::decay_t<decltype(d.params.default_value)>;
            st.plane.flags = FKB_PLANE_DEFAULT_VALUE;
            st.src_format = source_format_of<DV>();
            st.background[0] = (float)d.params.default_value.x; st.background[1] = (float)d.params.default_value.y;
            st.background[2] = (float)d.params.default_value.z;
            st.plane.crop_width = (int32_t)d.params.activeThreads.x; st.plane.crop_height = (int32_t)d.params.activeThreads.y;
            st.plane.src_width = d.params.activeThreads.x; st.plane.src_height = d.params.activeThreads.y;
        }
    }
};

/* computeCircularThreadIdx (memory_operations.h:436-446) */
inline int circular_plane(bool ascendent, int z, int first, int batch) {
    if (ascendent) { const int p = z + first; return p >= batch ? p - batch : p; }
    const int p = first - z;
    return p < 0 ? batch + p : p;
}
/* one plane of a tensor as the source of a plane that only moves it */
template <typename Op> struct TensorSource {
    static_assert(dependent_false<Op>::value, "fkb200: this tensor read is not on the accelerated path");
};
template <typename T> struct TensorSource<fk::TensorRead<T>> {
    template <typename Raw> static void fill(PlaneState& st, const Raw& t, int plane) {
        st.src_format = source_format_of<T>();
        st.plane.src = reinterpret_cast<const unsigned char*>(t.data) + (size_t)t.dims.plane_pitch * t.dims.color_planes * plane;
        st.plane.src_width = t.dims.width; st.plane.src_height = t.dims.height; st.plane.src_pitch = t.dims.pitch;
        st.plane.crop_x = 0; st.plane.crop_y = 0; st.plane.crop_width = (int32_t)t.dims.width; st.plane.crop_height = (int32_t)t.dims.height;
    }
};
/* TensorPack<float3> (memory_operations.h:257-289) reads what TensorSplit<float3> wrote: three float planes */
template <> struct TensorSource<fk::TensorPack<float3>> {
    template <typename Raw> static void fill(PlaneState& st, const Raw& t, int plane) {
        if (t.dims.pitch != t.dims.width * sizeof(float) || t.dims.plane_pitch != t.dims.pitch * t.dims.height || t.dims.color_planes != 3)
            throw std::runtime_error("fkb200: a planar tensor that is read back must be dense (pitch = width * 4, three colour planes)");
        st.raw_planar = true;
        st.src_format = FKB_SRC_F32X3;
        st.plane.src = reinterpret_cast<const unsigned char*>(t.data) + (size_t)t.dims.plane_pitch * 3 * plane;
        st.plane.src_width = t.dims.width; st.plane.src_height = t.dims.height; st.plane.src_pitch = t.dims.width * 12;
        st.plane.crop_x = 0; st.plane.crop_y = 0; st.plane.crop_width = (int32_t)t.dims.width; st.plane.crop_height = (int32_t)t.dims.height;
    }
};
/* CircularTensorRead<dir, Op, BATCH> (memory_operations.h:531-563): plane z reads tensor plane first -+ z */
template <fk::CircularDirection DIR, typename Op, int B> struct LowerFirst<fk::CircularTensorRead<DIR, Op, B>> {
    template <typename D> static void apply(std::vector<PlaneState>& states, const D& d) {
        states.reserve(B);
        for (int z = 0; z < B; ++z) {
            states.emplace_back();
            TensorSource<Op>::fill(states.back(), d.params.opData.params, circular_plane(DIR == fk::CircularDirection::Ascendent, z, d.params.first, B));
        }
    }
};
/* MidWrite<CircularTensorWrite<dir, WriteOp, BATCH>> (memory_operations.h:566-590): a second store of the value */
template <typename Op> struct CircularWriteTraits : std::false_type {};
template <fk::CircularDirection DIR, typename WOp, int B> struct CircularWriteTraits<fk::CircularTensorWrite<DIR, WOp, B>> : std::true_type {
    using Write = WOp;
    static constexpr bool ascendent = DIR == fk::CircularDirection::Ascendent;
    static constexpr int batch = B;
};

template <typename IOp> inline void lower_middle(std::vector<PlaneState>& states, const IOp& iop) {
    for (PlaneState& st : states) lower_compute<typename IOp::Operation>(st, iop);
}

inline bool same_sequence(const PlaneState& a, const fkb_sequence& q, const std::vector<fkb_op>& ops, int dst_format) {
    if (a.src_format != q.src_format || dst_format != q.dst_format || a.resize_mode != q.resize_mode) return false;
    if ((int)a.ops.size() != q.n_ops || (a.resize_mode == FKB_RESIZE_NONE ? 0 : a.n_pre_ops) != q.n_pre_ops) return false;
    if (std::memcmp(a.background, q.background, sizeof a.background) != 0) return false;
    if (a.border_mode != q.border_mode || a.deinterlace != q.deinterlace || std::memcmp(a.border_value, q.border_value, sizeof a.border_value) != 0 ||
        std::memcmp(a.transform, q.transform, sizeof a.transform) != 0) return false;
    for (size_t k = 0; k < ops.size(); ++k)
        if (a.ops[k].opcode != ops[k].opcode || std::memcmp(a.ops[k].p, ops[k].p, sizeof ops[k].p) != 0) return false;
    return true;
}

/* only_plane < 0: every plane of the chain; otherwise the chain as the reference's plane `only_plane` runs it (thread.z =
   only_plane): that plane of a batched read, or a single-image read, stored at that plane of the receiver */
template <typename First, typename... Rest>
inline LoweredPlan lower_planes(int only_plane, const First& first, const Rest&... rest) {
    static_assert(sizeof...(Rest) >= 1, "fkb200: a sender chain must be closed by a receiver");
    LoweredPlan plan;
    LowerFirst<typename First::Operation>::apply(plan.states, first);
    if (only_plane >= 0 && plan.states.size() > 1) {
        if ((size_t)only_plane >= plan.states.size()) throw std::runtime_error("fkb200: the sequence selected for a plane has fewer planes");
        PlaneState keep = plan.states[(size_t)only_plane];
        plan.states.assign(1, keep);
    }
    /* everything between the read and the receiver continues every plane; the last one is the receiver */
    Receiver recv, mid_recv;
    bool has_mid = false, mid_ascendent = true;
    int mid_first = 0, mid_batch = 1;
    size_t index = 0;
    auto visit = [&](const auto& iop) {
        using IOp = std::decay_t<decltype(iop)>;
        using Op = typename IOp::Operation;
        if (++index == sizeof...(Rest)) {
            if constexpr (fk::isWriteType<Op> && !CircularWriteTraits<Op>::value) recv = LowerWrite<Op>::apply(iop);
            else throw std::runtime_error("fkb200: the last operation must be a receiver");
        } else {
            if constexpr (CircularWriteTraits<Op>::value) {
                if (index + 1 != sizeof...(Rest)) throw std::runtime_error("fkb200: a mid-chain write anywhere but directly before the receiver is not on the accelerated path");
                mid_recv = LowerWrite<typename CircularWriteTraits<Op>::Write>::apply(iop.params.opData);
                has_mid = true; mid_ascendent = CircularWriteTraits<Op>::ascendent; mid_batch = CircularWriteTraits<Op>::batch;
                mid_first = iop.params.first;
            } else if constexpr (fk::isWriteType<Op>) throw std::runtime_error("fkb200: mid-chain writes are not on the accelerated path");
            else lower_middle(plan.states, iop);
        }
    };
    (visit(rest), ...);
    if (only_plane < 0 && recv.planes < plan.states.size()) throw std::runtime_error("fkb200: the receiver has fewer planes than the batch");
    if (only_plane >= 0 && recv.planes <= (size_t)only_plane) throw std::runtime_error("fkb200: the receiver has no such plane");
    if (has_mid && (mid_recv.dst_format != recv.dst_format || mid_recv.planes < (uint32_t)mid_batch))
        throw std::runtime_error("fkb200: the mid-chain write must use the receiver's layout and hold BATCH planes");
    for (size_t i = 0; i < plan.states.size(); ++i) {
        PlaneState& st = plan.states[i];
        const size_t z = only_plane >= 0 ? (size_t)only_plane : i;
        if (st.resize_mode == FKB_RESIZE_NONE) { st.plane.dst_width = (uint32_t)st.plane.crop_width; st.plane.dst_height = (uint32_t)st.plane.crop_height; }
        if (st.plane.dst_width > recv.width || st.plane.dst_height > recv.height)
            throw std::runtime_error("fkb200: the sender's output is larger than the receiver");
        int dst_format = recv.dst_format;
        uint32_t pitch = recv.pitch, channel_stride = recv.channel_stride;
        if (st.raw_planar) { /* moved as it lies: only into a receiver of the same dense planar layout, with nothing in between */
            if (!st.ops.empty() || st.resize_mode != FKB_RESIZE_NONE || recv.dst_format != FKB_DST_F32_PLANAR3 || recv.pitch != recv.width * 4u ||
                recv.channel_stride != recv.width * recv.height * 4u || st.plane.dst_width != recv.width || st.plane.dst_height != recv.height)
                throw std::runtime_error("fkb200: a planar tensor plane can only be moved into a dense TensorSplit receiver of the same size");
            dst_format = FKB_DST_F32X3_PACKED; pitch = recv.width * 12u; channel_stride = 0;
        }
        size_t s = 0;
        for (; s < plan.sequences.size(); ++s)
            if (same_sequence(st, plan.sequences[s], plan.sequence_ops[s], dst_format)) break;
        if (s == plan.sequences.size()) {
            fkb_sequence q{};
            q.src_format = st.src_format; q.dst_format = dst_format; q.resize_mode = st.resize_mode;
            q.n_ops = (int32_t)st.ops.size(); q.n_pre_ops = st.resize_mode == FKB_RESIZE_NONE ? 0 : st.n_pre_ops;
            std::memcpy(q.background, st.background, sizeof q.background);
            q.border_mode = st.border_mode; q.deinterlace = st.deinterlace;
            std::memcpy(q.border_value, st.border_value, sizeof q.border_value);
            std::memcpy(q.transform, st.transform, sizeof q.transform);
            plan.sequences.push_back(q);
            plan.sequence_ops.push_back(st.ops);
        }
        st.plane.sequence = (int32_t)s;
        st.plane.dst = static_cast<unsigned char*>(recv.data) + z * recv.plane_bytes;
        st.plane.dst_pitch = pitch;
        st.plane.dst_channel_stride = channel_stride;
        plan.planes.push_back(st.plane);
        if (has_mid) {
            fkb_plane second = st.plane;
            second.dst = static_cast<unsigned char*>(mid_recv.data) + (size_t)circular_plane(mid_ascendent, (int)z, mid_first, mid_batch) * mid_recv.plane_bytes;
            second.dst_pitch = mid_recv.pitch; second.dst_channel_stride = mid_recv.channel_stride;
            plan.planes.push_back(second);
        }
    }
    return plan;
}

template <typename First, typename... Rest>
inline LoweredPlan lower(const First& first, const Rest&... rest) { return lower_planes(-1, first, rest...); }

/* Several sequences in one launch (DivergentBatchTransformDPP, data_parallel_patterns.h:301-353): plane z runs the
   sequence whose 1-based number SequenceSelector::at(z) returns (:316-325); a plane no sequence claims does nothing. */
template <typename SequenceSelector, typename... Sequences>
inline LoweredPlan lower_divergent(const Sequences&... sequences) {
    size_t n_planes = 0;
    auto count = [&](const auto& seq) {
        const LoweredPlan all = fk::apply([](const auto&... iops) { return lower_planes(-1, iops...); }, seq.instantiableOperations);
        if (all.states.size() > n_planes) n_planes = all.states.size();
    };
    (count(sequences), ...);
    LoweredPlan plan;
    for (size_t z = 0; z < n_planes; ++z) {
        const unsigned chosen = SequenceSelector::at((unsigned)z);
        unsigned number = 0;
        auto take = [&](const auto& seq) {
            if (++number != chosen) return;
            LoweredPlan one = fk::apply([&](const auto&... iops) { return lower_planes((int)z, iops...); }, seq.instantiableOperations);
            for (fkb_plane p : one.planes) {
                const fkb_sequence& q = one.sequences[(size_t)p.sequence];
                const std::vector<fkb_op>& ops = one.sequence_ops[(size_t)p.sequence];
                size_t s = 0;
                for (; s < plan.sequences.size(); ++s) {
                    const fkb_sequence& e = plan.sequences[s];
                    if (e.src_format != q.src_format || e.dst_format != q.dst_format || e.resize_mode != q.resize_mode || e.n_ops != q.n_ops ||
                        e.n_pre_ops != q.n_pre_ops || e.border_mode != q.border_mode || e.deinterlace != q.deinterlace ||
                        std::memcmp(e.background, q.background, sizeof q.background) != 0 || std::memcmp(e.border_value, q.border_value, sizeof q.border_value) != 0 ||
                        std::memcmp(e.transform, q.transform, sizeof q.transform) != 0) continue;
                    bool same = true;
                    for (size_t k = 0; k < ops.size() && same; ++k)
                        same = plan.sequence_ops[s][k].opcode == ops[k].opcode && std::memcmp(plan.sequence_ops[s][k].p, ops[k].p, sizeof ops[k].p) == 0;
                    if (same) break;
                }
                if (s == plan.sequences.size()) { plan.sequences.push_back(q); plan.sequence_ops.push_back(ops); }
                p.sequence = (int32_t)s;
                plan.planes.push_back(p);
            }
        };
        (take(sequences), ...);
    }
    if (plan.planes.empty()) throw std::runtime_error("fkb200: no plane selects any of the sequences");
    return plan;
}

inline void check(int status) {
    if (status != FKB_OK)
        throw std::runtime_error(std::string("GPU Error: ") + (fkb_last_error()[0] ? fkb_last_error() : fkb_status_string(status)));
}

}  // namespace binding
}  // namespace fkb200

namespace fk {

/* The executor of the fkb200::TransformDPP tag: same shape as Executor<TransformDPP<ParArch::GPU_NVIDIA, TFEN>>
   (executors.h:245-293), with the launch replaced by a call into libfkb200. */
template <>
struct Executor<fkb200::TransformDPP> {
    FK_STATIC_STRUCT(Executor, Executor)
private:
    using Child = Executor<fkb200::TransformDPP>;
    using Parent = BaseExecutor<Child>;

    template <typename... IOps>
    FK_HOST_FUSE void executeOperations_helper(Stream_<ParArch::GPU_NVIDIA>& stream_, const IOps&... iOps) {
        fkb200::binding::LoweredPlan plan = fkb200::binding::lower(iOps...);
        const fkb_plan_desc desc = plan.desc();
        fkb200::binding::check(fkb_execute_async(&desc, stream_.getCUDAStream()));
    }
public:
    FK_HOST_FUSE ParArch parArch() { return ParArch::GPU_NVIDIA; }
    DECLARE_EXECUTOR_PARENT_IMPL
};

/* The executor that CircularTensor::update calls (core/data/circular_tensor.h:146) and the reference leaves undefined:
   several operation sequences, one launch, plane z running the sequence SequenceSelector::at(z) names. */
template <typename SequenceSelector>
struct Executor<DivergentBatchTransformDPP<ParArch::GPU_NVIDIA, SequenceSelector>> {
    FK_STATIC_STRUCT(Executor, Executor)
    template <typename... Sequences>
    FK_HOST_FUSE void executeOperations(const Stream_<ParArch::GPU_NVIDIA>& stream_, const Sequences&... sequences) {
        fkb200::binding::LoweredPlan plan = fkb200::binding::lower_divergent<SequenceSelector>(sequences...);
        const fkb_plan_desc desc = plan.desc();
        fkb200::binding::check(fkb_execute_async(&desc, stream_.getCUDAStream()));
    }
    FK_HOST_FUSE ParArch parArch() { return ParArch::GPU_NVIDIA; }
};
/* update() names the host variant in the other branch of a run-time test (:152), so it must exist to compile;
   this library has no CPU path */
template <typename SequenceSelector>
struct Executor<DivergentBatchTransformDPP<ParArch::CPU, SequenceSelector>> {
    FK_STATIC_STRUCT(Executor, Executor)
    template <typename StreamType, typename... Sequences>
    FK_HOST_FUSE void executeOperations(const StreamType&, const Sequences&...) {
        throw std::runtime_error("fkb200: divergent sequences run on device memory only (no CPU path)");
    }
    FK_HOST_FUSE ParArch parArch() { return ParArch::CPU; }
};

}  // namespace fk

#endif /* FKB200_EXECUTOR_H */
