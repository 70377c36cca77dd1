// Shared-memory swizzle atoms the intent selectors choose between (reference
// include/axp/swizzle.hpp:13-16: None, B32, B64, B128 as aliases of the stage
// protocol's SwizzleAtom types).  Here an atom carries the span in bytes and the
// two encodings the sm100 realizations need: the CUtensorMap swizzle enumerator and
// the layout code of the tcgen05 shared-memory matrix descriptor (bits 61-63).
#pragma once
#include <iro_cuda_ax_core.hpp>

namespace axp::swizzle {

template <int SpanBytes, int TensorMapEnum, int DescriptorCode>
struct Atom {
    static constexpr int span_bytes = SpanBytes;            // bytes of one swizzled row span (0: no swizzle)
    static constexpr int tensor_map_swizzle = TensorMapEnum;   // CU_TENSOR_MAP_SWIZZLE_{NONE,32B,64B,128B} = 0..3
    static constexpr int descriptor_code = DescriptorCode;     // tcgen05 descriptor: 0 none, 6 = 32 B, 4 = 64 B, 2 = 128 B
    static constexpr iro::util::u64 id = iro::util::mix_u64(iro::util::fnv1a_64_cstr("axp.swizzle.atom"), iro::util::u64(SpanBytes));
};

using None = Atom<0, 0, 0>;
using B32 = Atom<32, 1, 6>;
using B64 = Atom<64, 2, 4>;
using B128 = Atom<128, 3, 2>;

}  // namespace axp::swizzle
