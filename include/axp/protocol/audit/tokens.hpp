// Audit of the token lists on a contract's ports (reference include/axp/protocol/audit/tokens.hpp:35-80): a port that
// carries a tile must name visibility and liveness of its subject, an output port written by a warpgroup or a wider
// group must also name the synchronisation that publishes it; handles and scalars must be alive.
#pragma once
#include <iro_cuda_ax_core.hpp>

namespace axp::protocol::audit {

namespace detail {
template <class Port, bool IsInput = Port::is_input>
struct tokens_of {
    using type = typename Port::required;
};
template <class Port>
struct tokens_of<Port, false> {
    using type = typename Port::provided;
};
}  // namespace detail

template <class Port>
constexpr bool port_tokens_complete() {
    using tokens = typename detail::tokens_of<Port>::type;
    using subject = typename Port::subject;
    constexpr bool alive = iro::verify::has_token_kind_subject<tokens, iro::token::kind_alive, subject>();
    if constexpr (iro::contract::TilePayload<typename Port::payload>) {
        constexpr bool visible = iro::verify::has_token_kind_subject<tokens, iro::token::kind_visible_at, subject>();
        constexpr bool wide = iro::scope::min_scope_for_t<typename Port::exec_group>::level >= iro::scope::warpgroup::level;
        if constexpr (!Port::is_input && wide) {
            return visible && alive && iro::verify::has_token_kind_subject<tokens, iro::token::kind_sync_at, subject>();
        } else {
            return visible && alive;
        }
    } else {
        return alive;
    }
}

template <class Ports>
struct ports_complete;
template <class... Ps>
struct ports_complete<iro::util::type_list<Ps...>> : std::bool_constant<(port_tokens_complete<Ps>() && ...)> {};

template <class Contract>
constexpr bool contract_tokens_complete() {
    return ports_complete<typename Contract::inputs>::value && ports_complete<typename Contract::outputs>::value;
}

}  // namespace axp::protocol::audit
