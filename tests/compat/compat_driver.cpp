// Caller written against the reference's C++ launch interface (engine/mma_any/aq_bmma_op.h, engine/wmma_any/wmma_any.h,
// fastertransformer/.../abqgemm/abq_gemm_wrapper.h), compiled against include/abq_compat.hpp + libabq_b200.so instead.
// tests/test_gpu_compat_cpp.py builds it, feeds it operands as raw files and checks what it writes against the CPU oracle.
//
//   compat_driver <scenario> <dir> M N K
//     initexec   W2A8 signed planes: the named Init/Exec pairs FasterTransformer picks by M == 1 (abq_gemm_wrapper.cu:105-126), int32 out
//     wmma_any   W4A4 unsigned planes through launchWmmaAnyKernel as engine/test_w4a4_uint_wmma.cu:230 spells it, int32 out
//     wrapper    ABQGEMMWrapper(8, 2, true).gemm on fp16 activations with the workspace FasterTransformer allocates
//                (8 * tokens * K / 8 bytes, layers/FfnLayer.cc:670-673), fp16 out; scale_out is a float re-read as fp16
//     wrapper_u  the same with SIGNED = false (activations go through the planes in the caller's workspace)
//     wrapper_p  as wrapper, after ABQGEMMWrapper::prepare_weights (the library's extension: weights re-ordered once at load)
// Reads <dir>/x.bin, <dir>/w.bin (and scale.bin, scale_out.bin for the wrapper), writes <dir>/d.bin.  Exit code 0 = ran.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "abq_compat.hpp"

ABQ_COMPAT_DEFINE_CONFIG(AqBMMA_8x2xtrue_1x48x512_8x24x128_8x8x128_4, 8, 2, true)
ABQ_COMPAT_DEFINE_CONFIG(AqBMMA_8x2xtrue_8x48x256_32x48x128_8x8x128_5, 8, 2, true)

static std::vector<char> slurp(const std::string &path)
{
    FILE *f = std::fopen(path.c_str(), "rb");
    if (!f) {
        std::fprintf(stderr, "cannot open %s\n", path.c_str());
        std::exit(2);
    }
    std::fseek(f, 0, SEEK_END);
    long n = std::ftell(f);
    std::fseek(f, 0, SEEK_SET);
    std::vector<char> buf((size_t)n);
    if (n && std::fread(buf.data(), 1, (size_t)n, f) != (size_t)n)
        std::exit(2);
    std::fclose(f);
    return buf;
}

static void *to_device(const std::vector<char> &h)
{
    void *d = nullptr;
    if (cudaMalloc(&d, h.size() ? h.size() : 16) != cudaSuccess || cudaMemcpy(d, h.data(), h.size(), cudaMemcpyHostToDevice) != cudaSuccess) {
        std::fprintf(stderr, "device upload failed\n");
        std::exit(3);
    }
    return d;
}

static void dump(const std::string &path, const void *dev, size_t bytes)
{
    std::vector<char> h(bytes);
    if (cudaMemcpy(h.data(), dev, bytes, cudaMemcpyDeviceToHost) != cudaSuccess) {
        std::fprintf(stderr, "download failed: %s\n", cudaGetErrorString(cudaGetLastError()));
        std::exit(4);
    }
    FILE *f = std::fopen(path.c_str(), "wb");
    std::fwrite(h.data(), 1, bytes, f);
    std::fclose(f);
}

int main(int argc, char **argv)
{
    if (argc != 6) {
        std::fprintf(stderr, "usage: compat_driver <initexec|wmma_any|wrapper|wrapper_u|wrapper_p> <dir> M N K\n");
        return 1;
    }
    const std::string what = argv[1], dir = argv[2];
    const int M = std::atoi(argv[3]), N = std::atoi(argv[4]), K = std::atoi(argv[5]);
    cudaStream_t stream;
    cudaStreamCreate(&stream);
    void *x = to_device(slurp(dir + "/x.bin"));
    void *w = to_device(slurp(dir + "/w.bin"));

    if (what == "initexec") {
        int *D = nullptr;
        cudaMalloc(&D, (size_t)M * N * 4);
        cudaMemset(D, 0xff, (size_t)M * N * 4);
        AqBMMAInitFn_t init_fn;
        AqBMMAExecFn_t exec_fn;
        if (M == 1) {
            init_fn = AqBMMA_8x2xtrue_1x48x512_8x24x128_8x8x128_4_InitFn;
            exec_fn = AqBMMA_8x2xtrue_1x48x512_8x24x128_8x8x128_4_ExecFn;
        } else {
            init_fn = AqBMMA_8x2xtrue_8x48x256_32x48x128_8x8x128_5_InitFn;
            exec_fn = AqBMMA_8x2xtrue_8x48x256_32x48x128_8x8x128_5_ExecFn;
        }
        AqBMMAOpState state = (*init_fn)(reinterpret_cast<int *>(x), reinterpret_cast<int *>(w), M, N, K, D, nullptr, false);
        if (!state.initSuccess)
            return 5;
        (*exec_fn)(state, stream);
        (*exec_fn)(state, stream); // a state is launched many times (engine/test/test_mma/test_mma.h:127-140)
        if (cudaStreamSynchronize(stream) != cudaSuccess)
            return 6;
        // the reference refuses a bias (aq_bmma_op.h:79): so does the shim
        AqBMMAOpState bad = (*init_fn)(reinterpret_cast<int *>(x), reinterpret_cast<int *>(w), M, N, K, D, nullptr, true);
        if (bad.initSuccess)
            return 7;
        dump(dir + "/d.bin", D, (size_t)M * N * 4);
    } else if (what == "wmma_any") {
        int *D = nullptr;
        cudaMalloc(&D, (size_t)M * N * 4);
        cudaMemset(D, 0xff, (size_t)M * N * 4);
        AnyQuantParams params = { reinterpret_cast<const int *>(x), reinterpret_cast<const int *>(w), nullptr, D, false, M, N, K };
        cudaError_t err =
            launchWmmaAnyKernel<QuantType<4, 4, false>, ShapeBase<16, 16, 128>, ShapeBase<16, 32, 128>, ShapeBase<8, 8, 128>, 2>(params, stream);
        if (err != cudaSuccess || cudaStreamSynchronize(stream) != cudaSuccess)
            return 6;
        dump(dir + "/d.bin", D, (size_t)M * N * 4);
    } else if (what == "wrapper" || what == "wrapper_u" || what == "wrapper_p") {
        const bool is_signed = what != "wrapper_u";
        void *scale = to_device(slurp(dir + "/scale.bin"));         // float: activation quantiser scale
        void *scale_out = to_device(slurp(dir + "/scale_out.bin")); // float whose first two bytes are the fp16 output scale
        half *D = nullptr;
        cudaMalloc(&D, (size_t)M * N * 2);
        cudaMemset(D, 0xff, (size_t)M * N * 2);
        const size_t ws_bytes = (size_t)8 * M * K / 8; // what the FasterTransformer layers allocate: the activation planes only
        char *ws = nullptr;
        cudaMalloc(&ws, ws_bytes);
        ABQGEMMWrapper wrapper(8, 2, is_signed);
        if (what == "wrapper_p") {
            void *prepared = nullptr;
            const size_t nbytes = wrapper.prepared_weight_bytes(N, K);
            if (nbytes == 0 || cudaMalloc(&prepared, nbytes) != cudaSuccess ||
                !wrapper.prepare_weights(reinterpret_cast<const int *>(w), N, K, prepared, stream))
                return 9;
        }
        wrapper.gemm(M, N, K, reinterpret_cast<const half *>(x), reinterpret_cast<const int *>(w), nullptr, D,
                     reinterpret_cast<const float *>(scale), nullptr, reinterpret_cast<const float *>(scale_out), false, ws, ws_bytes, stream);
        if (cudaStreamSynchronize(stream) != cudaSuccess)
            return 6;
        dump(dir + "/d.bin", D, (size_t)M * N * 2);
        if (!is_signed) // the planes the pack step left in the caller's workspace are part of the contract
            dump(dir + "/planes.bin", ws, ws_bytes);
    } else {
        return 1;
    }
    if (cudaGetLastError() != cudaSuccess)
        return 8;
    return 0;
}
