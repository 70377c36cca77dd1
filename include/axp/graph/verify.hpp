// Structural verification of a selected graph (reference include/axp/graph/verify.hpp:36-84):
// every obligation has an id, the list has no duplicate, resources fit the capability
// (checked when the composition is formed) and every obligation binds to an sm100
// realization; and the contract flow of the list is closed (flow.hpp): every token an input port requires was provided
// by an earlier obligation, by the graph's externals or by a loop-carried token that the list provides again.
#pragma once
#include <iro_cuda_ax_core.hpp>

#include "../kits/sm100/index.hpp"
#include "flow.hpp"

namespace axp::graph {

template <class List>
struct no_duplicates;
template <>
struct no_duplicates<iro::util::type_list<>> : std::true_type {};
template <class T, class... Ts>
struct no_duplicates<iro::util::type_list<T, Ts...>>
    : std::bool_constant<!(std::is_same_v<T, Ts> || ...) && no_duplicates<iro::util::type_list<Ts...>>::value> {};

template <class List>
struct all_have_ids;
template <class... Ts>
struct all_have_ids<iro::util::type_list<Ts...>> : std::bool_constant<(iro::util::HasId<Ts> && ...)> {};

template <class G>
constexpr bool verify_structure() {
    using L = typename G::obligations;
    return L::size > 0 && all_have_ids<L>::value && no_duplicates<L>::value;
}

template <class G>
constexpr bool verify_contract_flow() {
    return axp::kit::sm100::binds_all<typename G::obligations>::value && G::smem_bytes <= G::cap::max_smem_bytes &&
           G::tmem_cols <= G::cap::tmem_columns && flow_closed<G>();
}

template <class G>
constexpr bool verify() {
    return verify_structure<G>() && verify_contract_flow<G>();
}

}  // namespace axp::graph
