// Audit of the token lists on a contract's ports.  Rule (the reference states it in
// include/axp/protocol/audit/tokens.hpp:35-80 and pins Tcgen05Mma and the tensor-memory moves with it,
// tests/compile/ax_asserts_primitives.cu:146-155,571-576):
//   tile payload, input port   -> the required list names visibility and liveness of the port's subject;
//   tile payload, output port  -> the provided list names both, and - when the port's execution group spans a
//                                 warpgroup or more - also the synchronisation that publishes the tile;
//   handle / scalar payload    -> liveness.
#pragma once
#include <iro_cuda_ax_core.hpp>

namespace axp::protocol::audit {

// The facts about one port the rule needs, as constants.
template <class Port>
struct port_audit {
    template <class P, bool In>
    struct list_of { using type = typename P::provided; };
    template <class P>
    struct list_of<P, true> { using type = typename P::required; };
    using tokens = typename list_of<Port, Port::is_input>::type;
    using subject = typename Port::subject;

    template <class Kind>
    static constexpr bool names = iro::verify::has_token_kind_subject<tokens, Kind, subject>();

    static constexpr bool carries_tile = iro::contract::TilePayload<typename Port::payload>;
    static constexpr bool wide_group = iro::scope::min_scope_for_t<typename Port::exec_group>::level >= iro::scope::warpgroup::level;
    static constexpr bool liveness = names<iro::token::kind_alive>;
    static constexpr bool visibility = names<iro::token::kind_visible_at>;
    static constexpr bool synchronisation = names<iro::token::kind_sync_at>;
    static constexpr bool complete =
        !carries_tile ? liveness : (visibility && liveness && (Port::is_input || !wide_group || synchronisation));
};

template <class Port>
constexpr bool port_tokens_complete() {
    return port_audit<Port>::complete;
}

template <class Ports>
inline constexpr bool every_port_complete = false;
template <class... Ps>
inline constexpr bool every_port_complete<iro::util::type_list<Ps...>> = (port_audit<Ps>::complete && ...);

template <class Contract>
constexpr bool contract_tokens_complete() {
    return every_port_complete<typename Contract::inputs> && every_port_complete<typename Contract::outputs>;
}

}  // namespace axp::protocol::audit
