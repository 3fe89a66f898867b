// Runs the reference-style chains of the configurations through include/fkb200_fk.hpp.
//   fk_shim_chains <dir>        reads <dir>/*.bin written by the Python test, runs on cuda:0, writes outputs
//   fk_shim_chains --host-only  exercises what needs no device: chain checks and the no-device error
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iostream>
#include <string>
#include <vector>

#include "fkb200_fk.hpp"

using namespace fkb200::fk;

static std::vector<unsigned char> read_file(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    if (!f) { std::cerr << "cannot read " << path << "\n"; std::exit(2); }
    return std::vector<unsigned char>((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
}
static void write_file(const std::string& path, const void* p, size_t n) {
    std::ofstream f(path, std::ios::binary);
    f.write(static_cast<const char*>(p), (std::streamsize)n);
}
#define CUDA_OK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { std::cerr << #x << ": " << cudaGetErrorString(e_) << "\n"; std::exit(3); } } while (0)
template <typename T> static T* to_device(const std::vector<unsigned char>& h) {
    void* d = nullptr; CUDA_OK(cudaMalloc(&d, h.size())); CUDA_OK(cudaMemcpy(d, h.data(), h.size(), cudaMemcpyHostToDevice)); return static_cast<T*>(d);
}
template <typename T> static T* device_zeros(size_t bytes) { void* d = nullptr; CUDA_OK(cudaMalloc(&d, bytes)); CUDA_OK(cudaMemset(d, 0, bytes)); return static_cast<T*>(d); }
static void download(const std::string& path, const void* d, size_t bytes) {
    std::vector<unsigned char> h(bytes); CUDA_OK(cudaMemcpy(h.data(), d, bytes, cudaMemcpyDeviceToHost)); write_file(path, h.data(), bytes);
}

static int host_only() {
    int failures = 0;
    auto expect_throw = [&](const char* what, auto&& fn, const char* needle) {
        try { fn(); std::cerr << "FAIL " << what << ": no exception\n"; ++failures; }
        catch (const std::runtime_error& e) {
            if (std::string(e.what()).find(needle) == std::string::npos) { std::cerr << "FAIL " << what << ": " << e.what() << "\n"; ++failures; }
            else std::cout << "ok " << what << ": " << e.what() << "\n";
        }
    };
    unsigned char dummy_in[64 * 3] = {0}; float dummy_out[64 * 3];
    const RawPtr2D<uchar3> img{reinterpret_cast<uchar3*>(dummy_in), 8, 8, 24};
    const RawPtr2D<float3> out{reinterpret_cast<float3*>(dummy_out), 8, 8, 96};
    // the reference would not compile Mul<float3> on a uchar3 value
    expect_throw("arithmetic on uchar3", [&] { (void)PerThreadRead<ND::_2D, uchar3>::build(img).then(Mul<float3>::build(make_set<float3>(2.f))); }, "not float3");
    // a float chain into a uchar3 receiver
    expect_throw("receiver type", [&] {
        Stream s;
        const RawPtr2D<uchar3> bad{reinterpret_cast<uchar3*>(dummy_in), 8, 8, 24};
        executeOperations<TransformDPP<>>(s, PerThreadRead<ND::_2D, uchar3>::build(img).then(Cast<uchar3, float3>::build()), PerThreadWrite<ND::_2D, uchar3>::build(bad));
    }, "does not match the receiver");
    // a border reader wraps the image read, not a crop of it
    expect_throw("border above crop", [&] {
        (void)BorderReader<BorderType::WRAP>::build(PerThreadRead<ND::_2D, uchar3>::build(img).then(Crop<>::build(Rect(1, 1, 4, 4))));
    }, "above a Crop");
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
        // no CPU fallback: the launch reports the missing device as an exception, like the reference's gpuErrchk
        expect_throw("no device", [&] {
            Stream s;
            executeOperations<TransformDPP<>>(s, PerThreadRead<ND::_2D, uchar3>::build(img).then(Cast<uchar3, float3>::build()), PerThreadWrite<ND::_2D, float3>::build(out));
        }, "no usable CUDA device");
    }
    return failures;
}

int main(int argc, char** argv) {
    if (argc < 2) { std::cerr << "usage: fk_shim_chains <dir> | --host-only\n"; return 2; }
    if (std::string(argv[1]) == "--host-only") return host_only();
    const std::string dir = argv[1];
    CUDA_OK(cudaSetDevice(0));
    cudaStream_t cs; CUDA_OK(cudaStreamCreate(&cs));
    {
        Stream stream(cs);

        // --- the README chain (reference tests/examples/readme_test_code.h:25-71), 384x216 frame ---
        const Size outputSize(60, 60);
        constexpr int BATCH = 5;
        uchar3* d_frame = to_device<uchar3>(read_file(dir + "/frame0.bin"));
        const RawPtr2D<uchar3> inputImage{d_frame, 384, 216, 384 * 3};
        float3* d_readme = device_zeros<float3>((size_t)BATCH * 60 * 60 * 12);
        const RawTensor<float3> output{d_readme, 60, 60, BATCH, 60 * 12};
        const std::array<Rect, BATCH> crops{Rect(0, 0, 34, 25), Rect(10, 10, 70, 15), Rect(20, 20, 60, 59), Rect(30, 30, 20, 23), Rect(40, 40, 12, 11)};
        const float3 backgroundColor{0.f, 0.f, 0.f};
        const float3 mulValue = make_set<float3>(1.4f), subValue = make_set<float3>(0.5f), divValue = make_set<float3>(255.f);
        const auto mySender = PerThreadRead<ND::_2D, uchar3>::build(inputImage)
            .then(Crop<>::build(crops))
            .then(Resize<InterpolationType::INTER_LINEAR, AspectRatio::PRESERVE_AR>::build(outputSize, backgroundColor))
            .then(Mul<float3>::build(mulValue))
            .then(Sub<float3>::build(subValue))
            .then(Div<float3>::build(divValue))
            .then(ColorConversion<ColorConversionCodes::COLOR_RGB2BGR, float3, float3>::build());
        const auto myReceiver = TensorWrite<float3>::build(output);
        executeOperations<TransformDPP<>>(stream, mySender, myReceiver);

        // --- batched crop -> resize -> normalise -> planar over two frames (configuration 3's chain) ---
        uchar3* d_frame1 = to_device<uchar3>(read_file(dir + "/frame1.bin"));
        const std::array<RawPtr2D<uchar3>, 4> frames{inputImage, RawPtr2D<uchar3>{d_frame1, 384, 216, 384 * 3}, inputImage, RawPtr2D<uchar3>{d_frame1, 384, 216, 384 * 3}};
        const std::array<Rect, 4> rects{Rect(5, 7, 200, 100), Rect(100, 50, 64, 160), Rect(0, 0, 384, 216), Rect(383, 215, 1, 1)};
        float* d_planar = device_zeros<float>((size_t)4 * 3 * 64 * 48 * 4);
        const auto normalise = PerThreadRead<ND::_2D, uchar3>::build(frames)
            .then(Crop<>::build(rects))
            .then(Resize<InterpolationType::INTER_LINEAR, AspectRatio::PRESERVE_AR>::build(Size(64, 48), backgroundColor))
            .then(Div<float3>::build(make_set<float3>(255.f)))
            .then(Sub<float3>::build(make_<float3>(0.485f, 0.456f, 0.406f)))
            .then(Div<float3>::build(make_<float3>(0.229f, 0.224f, 0.225f)));
        executeOperations<TransformDPP<>>(stream, normalise, TensorSplit<float3>::build(RawTensor<float>{d_planar, 64, 48, 4, 64 * 4}));

        // --- NV12 -> BT.709 RGB -> resize -> /255 (configuration 4's chain), two 96x54 frames ---
        unsigned char* d_nv0 = to_device<unsigned char>(read_file(dir + "/nv12_0.bin"));
        unsigned char* d_nv1 = to_device<unsigned char>(read_file(dir + "/nv12_1.bin"));
        const std::array<ImageNV12, 2> yuv{ImageNV12{d_nv0, 96, 54, 96}, ImageNV12{d_nv1, 96, 54, 96}};
        float3* d_rgb = device_zeros<float3>((size_t)2 * 40 * 22 * 12);
        const auto fromYUV = ReadYUV<PixelFormat::NV12>::build(yuv)
            .then(ConvertYUVToRGB<PixelFormat::NV12, ColorRange::Full, ColorPrimitives::bt709, false, float3>::build())
            .then(Resize<InterpolationType::INTER_LINEAR>::build(Size(40, 22)))
            .then(Div<float3>::build(make_set<float3>(255.f)));
        executeOperations<TransformDPP<>>(stream, fromYUV, TensorWrite<float3>::build(RawTensor<float3>{d_rgb, 40, 22, 2, 40 * 12}));

        // --- two different chains in one launch (divergent horizontal fusion) ---
        float3* d_div0 = device_zeros<float3>((size_t)384 * 216 * 12);
        uchar3* d_div1 = device_zeros<uchar3>((size_t)384 * 216 * 3);
        const auto seq0 = buildOperationSequence(
            PerThreadRead<ND::_2D, uchar3>::build(inputImage).then(Cast<uchar3, float3>::build()).then(Mul<float3>::build(mulValue)).then(Sub<float3>::build(subValue)),
            PerThreadWrite<ND::_2D, float3>::build(RawPtr2D<float3>{d_div0, 384, 216, 384 * 12}));
        const auto seq1 = buildOperationSequence(
            PerThreadRead<ND::_2D, uchar3>::build(RawPtr2D<uchar3>{d_frame1, 384, 216, 384 * 3})
                .then(ColorConversion<ColorConversionCodes::COLOR_RGB2BGR, uchar3, uchar3>::build())
                .then(Cast<uchar3, float3>::build()).then(Mul<float3>::build(mulValue)).then(SaturateCast<float3, uchar3>::build()),
            PerThreadWrite<ND::_2D, uchar3>::build(RawPtr2D<uchar3>{d_div1, 384, 216, 384 * 3}));
        executeDivergentOperations<TransformDPP<>>(stream, {seq0, seq1});

        // --- a padded crop under a reflecting border, resized (BorderReader -> Crop -> Resize) ---
        float3* d_border = device_zeros<float3>((size_t)70 * 45 * 12);
        const auto padded = BorderReader<BorderType::REFLECT_101>::build(PerThreadRead<ND::_2D, uchar3>::build(inputImage))
            .then(Crop<>::build(Rect(-20, -11, 430, 240)))
            .then(Resize<InterpolationType::INTER_LINEAR, AspectRatio::PRESERVE_AR_LEFT>::build(Size(70, 45), make_<float3>(1.f, 2.f, 3.f)));
        executeOperations<TransformDPP<>>(stream, padded, PerThreadWrite<ND::_2D, float3>::build(RawPtr2D<float3>{d_border, 70, 45, 70 * 12}));

        // --- a perspective warp, then Mul ---
        float3* d_warp = device_zeros<float3>((size_t)100 * 64 * 12);
        WarpingParameters<WarpType::Perspective> wp{{{0.9f, 0.1f, -2.0f}, {0.05f, 0.8f, 1.0f}, {0.002f, 0.001f, 1.0f}}, Size(100, 64)};
        const auto warped = PerThreadRead<ND::_2D, uchar3>::build(inputImage).then(Warping<WarpType::Perspective>::build(wp))
            .then(Mul<float3>::build(make_<float3>(1.f, 0.5f, 2.f)));
        executeOperations<TransformDPP<>>(stream, warped, PerThreadWrite<ND::_2D, float3>::build(RawPtr2D<float3>{d_warp, 100, 64, 100 * 12}));

        // --- Deinterlace<INTER_LINEAR> keeping the odd lines, then Mul ---
        float3* d_deint = device_zeros<float3>((size_t)384 * 216 * 12);
        const auto deint = Deinterlace<DeinterlaceType::INTER_LINEAR>::build(DeinterlaceLinear::USE_ODD, PerThreadRead<ND::_2D, uchar3>::build(inputImage))
            .then(Mul<float3>::build(make_<float3>(1.f, 0.5f, 2.f)));
        executeOperations<TransformDPP<>>(stream, deint, PerThreadWrite<ND::_2D, float3>::build(RawPtr2D<float3>{d_deint, 384, 216, 384 * 12}));

        // --- NV21 -> BT.601 RGB -> resize ---
        float3* d_rgb21 = device_zeros<float3>((size_t)2 * 40 * 22 * 12);
        const auto fromNV21 = ReadYUV<PixelFormat::NV21>::build(yuv)
            .then(ConvertYUVToRGB<PixelFormat::NV21, ColorRange::Full, ColorPrimitives::bt601, false, float3>::build())
            .then(Resize<InterpolationType::INTER_LINEAR>::build(Size(40, 22)))
            .then(Div<float3>::build(make_set<float3>(255.f)));
        executeOperations<TransformDPP<>>(stream, fromNV21, TensorWrite<float3>::build(RawTensor<float3>{d_rgb21, 40, 22, 2, 40 * 12}));

        // --- a circular tensor of the newest three normalised crops (CircularTensor::update, one launch per new image) ---
        CircularTensor<float, 3, 3, CircularTensorOrder::NewestFirst> window(64, 48, FKB_DST_F32_PLANAR3);
        for (int k = 0; k < 4; ++k) {
            const auto newest = PerThreadRead<ND::_2D, uchar3>::build(k % 2 ? RawPtr2D<uchar3>{d_frame1, 384, 216, 384 * 3} : inputImage)
                .then(Crop<>::build(rects[k]))
                .then(Resize<InterpolationType::INTER_LINEAR, AspectRatio::PRESERVE_AR>::build(Size(64, 48), backgroundColor))
                .then(Div<float3>::build(make_set<float3>(255.f)))
                .then(Sub<float3>::build(make_<float3>(0.485f, 0.456f, 0.406f)))
                .then(Div<float3>::build(make_<float3>(0.229f, 0.224f, 0.225f)));
            window.update(stream, newest, TensorSplit<float3>::build(window.ptr()));
        }

        stream.sync();   // everything above was asynchronous on the stream
        download(dir + "/out_window.bin", window.ptr().data, (size_t)3 * 3 * 64 * 48 * 4);
        download(dir + "/out_border.bin", d_border, (size_t)70 * 45 * 12);
        download(dir + "/out_warp.bin", d_warp, (size_t)100 * 64 * 12);
        download(dir + "/out_deint.bin", d_deint, (size_t)384 * 216 * 12);
        download(dir + "/out_nv21.bin", d_rgb21, (size_t)2 * 40 * 22 * 12);
        download(dir + "/out_readme.bin", d_readme, (size_t)BATCH * 60 * 60 * 12);
        download(dir + "/out_planar.bin", d_planar, (size_t)4 * 3 * 64 * 48 * 4);
        download(dir + "/out_nv12.bin", d_rgb, (size_t)2 * 40 * 22 * 12);
        download(dir + "/out_div0.bin", d_div0, (size_t)384 * 216 * 12);
        download(dir + "/out_div1.bin", d_div1, (size_t)384 * 216 * 3);
    }
    CUDA_OK(cudaStreamDestroy(cs));
    std::cout << "done\n";
    return 0;
}
