// Weight container of the INT4 servers: reader, writer and device upload.
//
// File format (writer: better-inference/gguf_convert.cpp:62-88; the same header is produced by
// scripts/quantize_awq_int4_8b.py:409-423; reader: server/inference_server_int4_batched.cu:32-45):
//   <prefix>.int4_t   int32 header [K, N, 16, K/16, 1], then N * K / 2 bytes: row n holds its K nibbles, two per byte,
//                     even k in the low nibble, value = nibble - 8
//   <prefix>.scale_t  int32 header [0, 0, 0, K/16, N], then N * (K/16) float32 scales, row-major
//   <name>.f32        raw float32 (norm weights), no header
// The reference reader trusts the files (no size or header check, unchecked fopen in places); this one validates the
// header fields against each other and against the file length and reports what is wrong through the return code.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <string>
#include <vector>

#include "../../include/blackwell_b200.h"

namespace {

// return codes of the file functions (negative: file problems; positive values are cudaError_t from the upload)
enum : int { kOk = 0, kErrOpen = -1, kErrShort = -2, kErrHeader = -3, kErrArg = -4, kErrWrite = -5 };

struct File {
    FILE* f;
    explicit File(const std::string& path, const char* mode) : f(fopen(path.c_str(), mode)) {}
    ~File() { if (f) fclose(f); }
};

long file_size(FILE* f) {
    const long cur = ftell(f);
    fseek(f, 0, SEEK_END);
    const long n = ftell(f);
    fseek(f, cur, SEEK_SET);
    return n;
}

int read_headers(const std::string& prefix, int* K, int* N) {
    File w(prefix + ".int4_t", "rb"), s(prefix + ".scale_t", "rb");
    if (!w.f || !s.f) return kErrOpen;
    int hw[5], hs[5];
    if (fread(hw, 4, 5, w.f) != 5 || fread(hs, 4, 5, s.f) != 5) return kErrShort;
    const int k = hw[0], n = hw[1];
    if (k <= 0 || n <= 0 || k % 16 != 0 || hw[2] != 16 || hw[3] != k / 16) return kErrHeader;
    if (hs[3] != k / 16 || hs[4] != n) return kErrHeader;
    if (file_size(w.f) != 20 + (long)((size_t)n * k / 2)) return kErrShort;
    if (file_size(s.f) != 20 + (long)((size_t)n * (k / 16) * 4)) return kErrShort;
    *K = k;
    *N = n;
    return kOk;
}

}  // namespace

extern "C" int bw_w4_file_write(const char* prefix, const uint8_t* packed, const float* scales, int K, int N) {
    if (!prefix || !packed || !scales || K <= 0 || N <= 0 || K % 16 != 0) return kErrArg;
    const int nkb = K / 16;
    {
        File f(std::string(prefix) + ".int4_t", "wb");
        if (!f.f) return kErrOpen;
        const int hdr[5] = {K, N, 16, nkb, 1};
        if (fwrite(hdr, 4, 5, f.f) != 5) return kErrWrite;
        const size_t n = (size_t)N * K / 2;
        if (fwrite(packed, 1, n, f.f) != n) return kErrWrite;
    }
    {
        File f(std::string(prefix) + ".scale_t", "wb");
        if (!f.f) return kErrOpen;
        const int hdr[5] = {0, 0, 0, nkb, N};
        if (fwrite(hdr, 4, 5, f.f) != 5) return kErrWrite;
        const size_t n = (size_t)N * nkb;
        if (fwrite(scales, 4, n, f.f) != n) return kErrWrite;
    }
    return kOk;
}

extern "C" int bw_w4_file_dims(const char* prefix, int* K_out, int* N_out) {
    if (!prefix || !K_out || !N_out) return kErrArg;
    return read_headers(prefix, K_out, N_out);
}

extern "C" int bw_w4_file_read(const char* prefix, uint8_t* packed_out, float* scales_out, int K, int N) {
    if (!prefix || !packed_out || !scales_out) return kErrArg;
    int k = 0, n = 0;
    const int e = read_headers(prefix, &k, &n);
    if (e != kOk) return e;
    if (k != K || n != N) return kErrArg;
    File w(std::string(prefix) + ".int4_t", "rb"), s(std::string(prefix) + ".scale_t", "rb");
    if (!w.f || !s.f) return kErrOpen;
    fseek(w.f, 20, SEEK_SET);
    fseek(s.f, 20, SEEK_SET);
    const size_t nb = (size_t)N * K / 2, ns = (size_t)N * (K / 16);
    if (fread(packed_out, 1, nb, w.f) != nb) return kErrShort;
    if (fread(scales_out, 4, ns, s.f) != ns) return kErrShort;
    return kOk;
}

// The device-side container: what the reference keeps per projection as DevW4 {K, N, d, sc}
// (server/inference_server_int4_batched.cu:31), plus the binary16 copy of the scales the W4A8 entry points take.
extern "C" int bw_w4_file_upload(const char* prefix, int want_f32_scales, int want_f16_scales, bw_dev_w4* out) {
    if (!prefix || !out) return kErrArg;
    memset(out, 0, sizeof(*out));
    int K = 0, N = 0;
    int e = read_headers(prefix, &K, &N);
    if (e != kOk) return e;
    const size_t nb = (size_t)N * K / 2, ns = (size_t)N * (K / 16);
    std::vector<uint8_t> hp(nb);
    std::vector<float> hs(ns);
    e = bw_w4_file_read(prefix, hp.data(), hs.data(), K, N);
    if (e != kOk) return e;
    out->K = K;
    out->N = N;
    cudaError_t ce = cudaMalloc(reinterpret_cast<void**>(&out->packed), nb);
    if (ce == cudaSuccess) ce = cudaMemcpy(out->packed, hp.data(), nb, cudaMemcpyHostToDevice);
    if (ce == cudaSuccess && want_f32_scales) {
        ce = cudaMalloc(reinterpret_cast<void**>(&out->scale_f32), ns * 4);
        if (ce == cudaSuccess) ce = cudaMemcpy(out->scale_f32, hs.data(), ns * 4, cudaMemcpyHostToDevice);
    }
    if (ce == cudaSuccess && want_f16_scales) {
        std::vector<uint16_t> h16(ns);
        for (size_t i = 0; i < ns; ++i) {
            const __half h = __float2half_rn(hs[i]);
            memcpy(&h16[i], &h, 2);
        }
        ce = cudaMalloc(reinterpret_cast<void**>(&out->scale_f16), ns * 2);
        if (ce == cudaSuccess) ce = cudaMemcpy(out->scale_f16, h16.data(), ns * 2, cudaMemcpyHostToDevice);
    }
    if (ce != cudaSuccess) {
        bw_w4_free(out);
        return (int)ce;
    }
    return kOk;
}

extern "C" int bw_w4_free(bw_dev_w4* w) {
    if (!w) return kErrArg;
    if (w->packed) cudaFree(w->packed);
    if (w->scale_f32) cudaFree(w->scale_f32);
    if (w->scale_f16) cudaFree(w->scale_f16);
    memset(w, 0, sizeof(*w));
    return kOk;
}

extern "C" int bw_f32_file_write(const char* path, const float* data, size_t n) {
    if (!path || !data) return kErrArg;
    File f(path, "wb");
    if (!f.f) return kErrOpen;
    return fwrite(data, 4, n, f.f) == n ? kOk : kErrWrite;
}

extern "C" int bw_f32_file_read(const char* path, float* data_out, size_t n) {
    if (!path || !data_out) return kErrArg;
    File f(path, "rb");
    if (!f.f) return kErrOpen;
    if (file_size(f.f) != (long)(n * 4)) return kErrShort;
    return fread(data_out, 4, n, f.f) == n ? kOk : kErrShort;
}
