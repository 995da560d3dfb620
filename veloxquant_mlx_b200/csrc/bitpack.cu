// LSB-first packing / unpacking of flat uint8 code arrays, 1, 2 or 4 bits per code.
// One thread per packed byte (pack) or per code (unpack); the tail of a ragged array is
// zero-filled in the last byte.
#include <algorithm>

#include "common.cuh"

namespace vq {

__global__ void bit_pack_kernel(const uint8_t *__restrict__ codes, int64_t n, int bits,
                                uint8_t *__restrict__ packed, int64_t n_bytes) {
    const int per = 8 / bits;
    const uint32_t mask = (1u << bits) - 1u;
    for (int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; j < n_bytes;
         j += (int64_t)gridDim.x * blockDim.x) {
        uint32_t byte = 0;
        for (int k = 0; k < per; ++k) {
            const int64_t i = j * per + k;
            if (i < n) byte |= (codes[i] & mask) << (k * bits);
        }
        packed[j] = (uint8_t)byte;
    }
}

__global__ void bit_unpack_kernel(const uint8_t *__restrict__ packed, int64_t n, int bits,
                                  uint8_t *__restrict__ codes) {
    const int per = 8 / bits;
    const uint32_t mask = (1u << bits) - 1u;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x)
        codes[i] = (uint8_t)((packed[i / per] >> ((i % per) * bits)) & mask);
}

}  // namespace vq

extern "C" int32_t vq_bit_pack(const uint8_t *codes, int64_t n, int32_t bits, uint8_t *packed, void *stream) {
    using namespace vq;
    VQ_REQUIRE(bits == 1 || bits == 2 || bits == 4, VQ_ERR_SHAPE, "bit_pack: bits must be 1, 2 or 4, got %d", bits);
    VQ_REQUIRE(n >= 0, VQ_ERR_SHAPE, "bit_pack: n must be >= 0");
    if (n == 0) return VQ_OK;
    const int64_t n_bytes = ceil_div(n * bits, 8);
    const unsigned blocks = (unsigned)std::min<int64_t>(ceil_div(n_bytes, 256), 148 * 16);
    bit_pack_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(codes, n, bits, packed, n_bytes);
    VQ_CHECK_LAUNCH("bit_pack_kernel");
    return VQ_OK;
}

extern "C" int32_t vq_bit_unpack(const uint8_t *packed, int64_t n, int32_t bits, uint8_t *codes, void *stream) {
    using namespace vq;
    VQ_REQUIRE(bits == 1 || bits == 2 || bits == 4, VQ_ERR_SHAPE, "bit_unpack: bits must be 1, 2 or 4, got %d", bits);
    VQ_REQUIRE(n >= 0, VQ_ERR_SHAPE, "bit_unpack: n must be >= 0");
    if (n == 0) return VQ_OK;
    const unsigned blocks = (unsigned)std::min<int64_t>(ceil_div(n, 256), 148 * 16);
    bit_unpack_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(packed, n, bits, codes);
    VQ_CHECK_LAUNCH("bit_unpack_kernel");
    return VQ_OK;
}
