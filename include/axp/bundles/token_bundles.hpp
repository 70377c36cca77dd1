// Token bundles: the token lists that ports of tile-moving obligations carry (reference
// include/axp/bundles/token_bundles.hpp:17-100).  A tile that an execution group reads must be visible to the smallest
// scope containing that group and stay alive while it is used; when that scope is a warpgroup or wider, the hand-over
// also needs a synchronisation of that scope (a barrier phase, an mbarrier, a tcgen05.commit).
#pragma once
#include <iro_cuda_ax_core.hpp>

namespace axp::bundle {

namespace detail {
template <class Subject, class ExecGroup, class Lifetime, bool Sync = (iro::scope::min_scope_for_t<ExecGroup>::level >= iro::scope::warpgroup::level)>
struct tile_tokens {
    using type = iro::util::type_list<iro::token::visible_at<Subject, iro::scope::min_scope_for_t<ExecGroup>>,
                                      iro::token::alive<Subject, Lifetime>>;
};
template <class Subject, class ExecGroup, class Lifetime>
struct tile_tokens<Subject, ExecGroup, Lifetime, true> {
    using type = iro::util::type_list<iro::token::visible_at<Subject, iro::scope::min_scope_for_t<ExecGroup>>,
                                      iro::token::alive<Subject, Lifetime>,
                                      iro::token::sync_at<Subject, iro::scope::min_scope_for_t<ExecGroup>>>;
};
}  // namespace detail

// required by an input port that reads a tile
template <class Subject, class ExecGroup, class Lifetime>
using TileInTokens = typename detail::tile_tokens<Subject, ExecGroup, Lifetime>::type;
// provided by an output port that wrote a tile
template <class Subject, class ExecGroup, class Lifetime>
using TileOutTokens = typename detail::tile_tokens<Subject, ExecGroup, Lifetime>::type;
// handles and scalars only have to exist
template <class Subject, class Lifetime>
using ValueLive = iro::util::type_list<iro::token::alive<Subject, Lifetime>>;

}  // namespace axp::bundle
