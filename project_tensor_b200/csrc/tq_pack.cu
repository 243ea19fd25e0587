// Conversions between the packed device layouts and the reference's array fields
// (indices: uint8 [n][d]; qjl: int8 [n][d] holding +1 / -1; _quant.py:156-169).
#include "tq_common.cuh"

namespace {

__global__ void unpack_codes_kernel(const uint32_t* __restrict__ codes, int64_t n, int d, int bits, int words,
                                    uint8_t* __restrict__ out) {
    const int64_t total = n * d;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / d;
        const int j = (int)(i - row * d);
        out[i] = (uint8_t)tq_get_code(codes + row * words, j, bits);
    }
}

__global__ void pack_codes_kernel(const uint8_t* __restrict__ in, int64_t n, int d, int bits, int words,
                                  uint32_t* __restrict__ codes) {
    const int64_t total = n * words;
    const uint32_t mask = (1u << bits) - 1u;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / words;
        const int w = (int)(i - row * words);
        const uint8_t* src = in + row * d;
        const int lo_bit = w * 32;
        uint32_t v = 0;
        for (int j = lo_bit / bits; j < d && j * bits < lo_bit + 32; ++j) {
            const int sh = j * bits - lo_bit;
            const uint32_t c = src[j] & mask;
            v |= sh >= 0 ? (c << sh) : (c >> (-sh));
        }
        codes[i] = v;
    }
}

__global__ void unpack_signs_kernel(const uint32_t* __restrict__ signs, int64_t n, int d, int words,
                                    int8_t* __restrict__ out) {
    const int64_t total = n * d;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / d;
        const int j = (int)(i - row * d);
        out[i] = ((signs[row * words + (j >> 5)] >> tq_sign_bitpos(j)) & 1u) ? (int8_t)1 : (int8_t)-1;
    }
}

__global__ void pack_signs_kernel(const int8_t* __restrict__ in, int64_t n, int d, int words,
                                  uint32_t* __restrict__ signs) {
    const int64_t total = n * words;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / words;
        const int w = (int)(i - row * words);
        uint32_t v = 0;
        for (int b = 0; b < 32; ++b) {
            const int j = w * 32 + b;
            if (j < d && in[row * d + j] >= 0) v |= 1u << tq_sign_bitpos(j);
        }
        signs[i] = v;
    }
}

int blocks_for(int64_t total) {
    int64_t b = (total + 255) / 256;
    if (b > 148 * 32) b = 148 * 32;
    return b < 1 ? 1 : (int)b;
}

}  // namespace

int tq_launch_unpack_codes(const tq_plan* p, const uint32_t* codes, int64_t n, uint8_t* out, cudaStream_t st) {
    if (n == 0) return TQ_OK;
    unpack_codes_kernel<<<blocks_for(n * p->dev.d), 256, 0, st>>>(codes, n, p->dev.d, p->dev.bits, p->dev.code_words, out); tq_count_launch();
    TQ_CUDA_TRY(cudaGetLastError());
    return TQ_OK;
}
int tq_launch_pack_codes(const tq_plan* p, const uint8_t* in, int64_t n, uint32_t* codes, cudaStream_t st) {
    if (n == 0) return TQ_OK;
    pack_codes_kernel<<<blocks_for(n * p->dev.code_words), 256, 0, st>>>(in, n, p->dev.d, p->dev.bits, p->dev.code_words, codes); tq_count_launch();
    TQ_CUDA_TRY(cudaGetLastError());
    return TQ_OK;
}
int tq_launch_unpack_signs(const tq_plan* p, const uint32_t* signs, int64_t n, int8_t* out, cudaStream_t st) {
    if (n == 0) return TQ_OK;
    unpack_signs_kernel<<<blocks_for(n * p->dev.d), 256, 0, st>>>(signs, n, p->dev.d, p->dev.sign_words, out); tq_count_launch();
    TQ_CUDA_TRY(cudaGetLastError());
    return TQ_OK;
}
int tq_launch_pack_signs(const tq_plan* p, const int8_t* in, int64_t n, uint32_t* signs, cudaStream_t st) {
    if (n == 0) return TQ_OK;
    pack_signs_kernel<<<blocks_for(n * p->dev.sign_words), 256, 0, st>>>(in, n, p->dev.d, p->dev.sign_words, signs); tq_count_launch();
    TQ_CUDA_TRY(cudaGetLastError());
    return TQ_OK;
}
