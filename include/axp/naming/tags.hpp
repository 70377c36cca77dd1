// Subject tags (reference include/axp/naming/tags.hpp:7-41): stable ids that
// name the operands a pattern talks about.
#pragma once
#include <iro_cuda_ax_core.hpp>

namespace axp::tag {
#define AXP_TAG(name) \
    struct name { static constexpr auto id = iro::util::fnv1a_64_cstr("axp.tag." #name); }
AXP_TAG(A);
AXP_TAG(B);
AXP_TAG(C);
AXP_TAG(O);
AXP_TAG(Acc);
AXP_TAG(Q);
AXP_TAG(K);
AXP_TAG(V);
AXP_TAG(S);
AXP_TAG(P);
AXP_TAG(ScaleA);
AXP_TAG(ScaleB);
AXP_TAG(Lse);
AXP_TAG(State);
#undef AXP_TAG
}  // namespace axp::tag
