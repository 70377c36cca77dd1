// Contract flow of a graph: walking the obligation list in order, every token that an input port requires must have
// been provided before it - by an output port of an earlier obligation, by the graph's externals (what the caller
// hands to the kernel: global tensors, scalars), or by a loop-carried token (state that the previous pass over the
// same list left behind, e.g. the attention accumulator published by the last P.V commit).  Loop-carried tokens are
// not free: at the end of the list every one of them must have been provided again by an obligation of the list.
// "Provided" means same kind and subject at a scope / lifetime at least as wide (iro::verify::satisfies_v).
//
// The reference checks the same property edge by edge while it composes (iro::compose edges,
// include/iro_cuda_ax_core.hpp:3801-3854, with the token audit of include/axp/protocol/audit/tokens.hpp); here the
// graph is a list, so the check is one walk.
#pragma once
#include <iro_cuda_ax_core.hpp>

#include "../protocol/audit/tokens.hpp"

namespace axp::graph {

namespace detail {

using iro::util::concat_t;
using iro::util::type_list;

// all tokens that the ports of a list require / provide
template <class Ports>
struct required_of;
template <class... Ps>
struct required_of<type_list<Ps...>> {
    template <class... Ls>
    struct fold {
        using type = type_list<>;
    };
    template <class L, class... Ls>
    struct fold<L, Ls...> {
        using type = concat_t<L, typename fold<Ls...>::type>;
    };
    using type = typename fold<typename Ps::required...>::type;
};
template <class Ports>
struct provided_of;
template <class... Ps>
struct provided_of<type_list<Ps...>> {
    template <class... Ls>
    struct fold {
        using type = type_list<>;
    };
    template <class L, class... Ls>
    struct fold<L, Ls...> {
        using type = concat_t<L, typename fold<Ls...>::type>;
    };
    using type = typename fold<typename Ps::provided...>::type;
};

template <class Available, class Needs>
struct all_satisfied;
template <class Available, class... Ns>
struct all_satisfied<Available, type_list<Ns...>> : std::bool_constant<(iro::verify::satisfies_v<Available, Ns> && ...)> {};

// Walk: `Given` = externals + carried (never grows), `Made` = tokens provided by the obligations seen so far.
// `index` of the first obligation with an unmet requirement, or -1.
template <class Obligations, class Given, class Made, int Index>
struct walk;
template <class Given, class Made, int Index>
struct walk<type_list<>, Given, Made, Index> {
    static constexpr int first_unmet = -1;
    using made = Made;
};
template <class O, class... Os, class Given, class Made, int Index>
struct walk<type_list<O, Os...>, Given, Made, Index> {
    using needs = typename required_of<typename O::inputs>::type;
    static constexpr bool ok = all_satisfied<concat_t<Given, Made>, needs>::value;
    using next = walk<type_list<Os...>, Given, concat_t<Made, typename provided_of<typename O::outputs>::type>, Index + 1>;
    static constexpr int first_unmet = ok ? next::first_unmet : Index;
    using made = typename next::made;
};

template <class List>
struct contracts_complete;
template <class... Os>
struct contracts_complete<type_list<Os...>> : std::bool_constant<(axp::protocol::audit::contract_tokens_complete<Os>() && ...)> {};

}  // namespace detail

// Everything the caller hands over for a global tensor or a scalar: visible to the device, alive for the kernel,
// ordered before the launch.
template <class Subject>
using external_tokens = iro::util::type_list<iro::token::visible_at<Subject, iro::scope::device>,
                                             iro::token::alive<Subject, iro::token::lifetime::kernel>,
                                             iro::token::sync_at<Subject, iro::scope::device>>;

template <class Obligations, class External, class Carried = iro::util::type_list<>>
struct flow {
    using w = detail::walk<Obligations, iro::util::concat_t<External, Carried>, iro::util::type_list<>, 0>;
    // index (in the obligation list) of the first obligation one of whose required tokens nothing provided; -1 if none
    static constexpr int first_unmet = w::first_unmet;
    // every loop-carried token is provided again by the list itself
    static constexpr bool carried_closed = detail::all_satisfied<typename w::made, Carried>::value;
    // every port of every obligation names the tokens its payload needs
    static constexpr bool ports_complete = detail::contracts_complete<Obligations>::value;
    static constexpr bool closed = first_unmet == -1 && carried_closed && ports_complete;
};

// G exposes `obligations`, `external` and `carried`.
template <class G>
constexpr bool flow_closed() {
    return flow<typename G::obligations, typename G::external, typename G::carried>::closed;
}

}  // namespace axp::graph
