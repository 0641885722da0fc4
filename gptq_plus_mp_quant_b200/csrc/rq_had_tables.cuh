// Sign tables of the K x K Hadamard matrices of orders 12, 20 and 28 (written by make_had_header.py; do not
// edit): bit c of had_row<K>(r) is set where entry (r, c) is +1.
#pragma once

#include <stdint.h>

namespace rq {
namespace fwht {

template <int K> __host__ __device__ constexpr uint32_t had_row(int r);
template <> __host__ __device__ constexpr uint32_t had_row<12>(int r) {
    constexpr uint32_t t[12] = {
        0x00000001u, 0x00000b8bu, 0x00000717u, 0x00000e2du, 0x00000c5bu, 0x000008b7u,
        0x0000016fu, 0x000002ddu, 0x000005b9u, 0x00000b71u, 0x000006e3u, 0x00000dc5u,
    };
    return t[r];
}
template <> __host__ __device__ constexpr uint32_t had_row<20>(int r) {
    constexpr uint32_t t[20] = {
        0x00000001u, 0x0009ea1bu, 0x0003d437u, 0x0007a86du, 0x000f50d9u, 0x000ea1b3u,
        0x000d4367u, 0x000a86cfu, 0x00050d9fu, 0x000a1b3du, 0x0004367bu, 0x00086cf5u,
        0x0000d9ebu, 0x0001b3d5u, 0x000367a9u, 0x0006cf51u, 0x000d9ea1u, 0x000b3d43u,
        0x00067a87u, 0x000cf50du,
    };
    return t[r];
}
template <> __host__ __device__ constexpr uint32_t had_row<28>(int r) {
    constexpr uint32_t t[28] = {
        0x0fffbfffu, 0x0b0d6c37u, 0x061ad86fu, 0x0c3570ddu, 0x086ae1bbu, 0x00d5c377u,
        0x01ab46edu, 0x03564dd9u, 0x06ac5bb1u, 0x0d587761u, 0x0ab0eec3u, 0x0561dd87u,
        0x0ac37b0du, 0x0586f61bu, 0x00003ffeu, 0x04f22c35u, 0x09e4186bu, 0x03c8b0d5u,
        0x079121abu, 0x0f220357u, 0x0e4486adu, 0x0c898d59u, 0x09139ab1u, 0x0227b561u,
        0x044f2ac3u, 0x089e1587u, 0x013cab0du, 0x0279161bu,
    };
    return t[r];
}

}  // namespace fwht
}  // namespace rq
