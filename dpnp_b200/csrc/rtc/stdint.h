// Stand-in for <stdint.h> when a fused chain is compiled at run time (no host headers there):
// the fixed-width types come from the CUDA C++ standard library.
#pragma once
#include <cuda/std/cstdint>
using cuda::std::int8_t;
using cuda::std::int16_t;
using cuda::std::int32_t;
using cuda::std::int64_t;
using cuda::std::uint8_t;
using cuda::std::uint16_t;
using cuda::std::uint32_t;
using cuda::std::uint64_t;
using cuda::std::uintptr_t;
using cuda::std::intptr_t;
