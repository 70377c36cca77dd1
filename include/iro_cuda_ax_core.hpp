// Contract substrate for the sm100 gemm / attention path: stable ids, type
// lists, element and recipe descriptors, capabilities, obligations, realization
// lookup and a resource-checked composition.
//
// This is a from-scratch, path-sized restatement of the vocabulary that the
// reference keeps in include/iro_cuda_ax_core.hpp (ids :245-262, recipes
// :2608-2758, obligations/realizations :3255-3300, caps :3308-3350, budgets
// :3356-3378, composition :3801-3854, lookup :3862-4031, elems :4106-4284).  It
// keeps the same names and meanings for everything the L4 presets, the L3
// registry and the sm100 kit need, and nothing else.  The id helpers are
// constexpr (not consteval), so the headers build with g++ 13 and nvcc 12.9.
#pragma once

#include <cstddef>
#include <cstdint>
#include <type_traits>

namespace iro::util {

using u64 = std::uint64_t;

// FNV-1a 64-bit of a NUL-terminated string (reference core:245-252).
constexpr u64 fnv1a_64_cstr(const char* s) {
    u64 h = 14695981039346656037ULL;
    for (; *s; ++s) {
        h ^= static_cast<unsigned char>(*s);
        h *= 1099511628211ULL;
    }
    return h;
}

// splitmix-style mix of two words (reference core:255-262).
constexpr u64 mix_u64(u64 h, u64 x) {
    x += 0x9e3779b97f4a7c15ULL;
    x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ULL;
    x = (x ^ (x >> 27)) * 0x94d049bb133111ebULL;
    x = x ^ (x >> 31);
    return h ^ x;
}

template <class... Ts>
struct type_list {
    static constexpr std::size_t size = sizeof...(Ts);
};

template <class A, class B>
struct concat;
template <class... As, class... Bs>
struct concat<type_list<As...>, type_list<Bs...>> {
    using type = type_list<As..., Bs...>;
};
template <class A, class B>
using concat_t = typename concat<A, B>::type;

// first element of a non-empty list
template <class List>
struct front;
template <class T, class... Ts>
struct front<type_list<T, Ts...>> {
    using type = T;
};
template <class List>
using front_t = typename front<List>::type;

template <class T, class List>
struct contains;
template <class T, class... Ts>
struct contains<T, type_list<Ts...>> : std::bool_constant<(std::is_same_v<T, Ts> || ...)> {};

template <class T>
concept HasId = requires { { T::id } -> std::convertible_to<u64>; };

// order-sensitive hash of the ids of a list (reference core:264-291)
template <class List>
struct hash_list;
template <class... Ts>
struct hash_list<type_list<Ts...>> {
    static_assert((HasId<Ts> && ...), "hash_list requires HasId elements");
    static constexpr u64 value = [] {
        u64 h = fnv1a_64_cstr("iro.util.hash_list");
        ((h = mix_u64(h, static_cast<u64>(Ts::id))), ...);
        return h;
    }();
};

}  // namespace iro::util

// ------------------------------------------------------------------ elements ----
namespace iro::elem {
#define IRO_ELEM(name, nbytes)                                                     \
    struct name {                                                                  \
        static constexpr int bytes = nbytes;                                       \
        static constexpr iro::util::u64 id = iro::util::fnv1a_64_cstr("iro.elem." #name); \
    }
IRO_ELEM(f32, 4);
IRO_ELEM(f16, 2);
IRO_ELEM(bf16, 2);
IRO_ELEM(e4m3, 1);
IRO_ELEM(e5m2, 1);
#undef IRO_ELEM
}  // namespace iro::elem

// ------------------------------------------------------------------- recipes ----
namespace iro::recipe {

struct Fast { static constexpr iro::util::u64 id = iro::util::fnv1a_64_cstr("iro.recipe.math.fast"); };
struct Accurate { static constexpr iro::util::u64 id = iro::util::fnv1a_64_cstr("iro.recipe.math.accurate"); };

// FP8 conversion policies (reference core:2634-2658): saturate clamps to the
// largest finite value before encoding.
struct fp8_native { static constexpr iro::util::u64 id = iro::util::fnv1a_64_cstr("iro.recipe.fp8.native"); };
struct fp8_saturate { static constexpr iro::util::u64 id = iro::util::fnv1a_64_cstr("iro.recipe.fp8.saturate"); };

// One input element type (reference `Precision`).
template <class In, class Acc, class Out, int Vec, class Math>
struct Precision {
    using in = In;
    using in_a = In;
    using in_b = In;
    using acc = Acc;
    using out = Out;
    using math = Math;
    using fp8_policy = fp8_native;
    using scale_a = void;
    using scale_b = void;
    static constexpr int vec = Vec;
    static constexpr int scale_vec_a = 0;
    static constexpr int scale_vec_b = 0;
    static constexpr bool has_scales = false;
    static constexpr iro::util::u64 id = iro::util::mix_u64(
        iro::util::fnv1a_64_cstr("iro.recipe.precision"),
        iro::util::mix_u64(In::id, iro::util::mix_u64(Acc::id, iro::util::mix_u64(Out::id, Math::id))));
};

// Separate A/B element types with optional operand scales (reference
// `PrecisionAB`, core:2711-2758).  On sm100 the scale vectors mean: ScaleVecA =
// rows of A sharing one K-block scale vector entry (1 = one scale per row per
// 128-wide K block), ScaleVecB = B rows per scale (128 = one scale per 128x128
// block); the scales multiply the fp32 partial sum of the K block.
template <class ElemA, class ElemB, class Acc, class Out, int Vec, class Math, class Fp8Policy = fp8_native,
          class ScaleElemA = void, int ScaleVecA = 0, class ScaleElemB = void, int ScaleVecB = 0>
struct PrecisionAB {
    using in = ElemA;
    using in_a = ElemA;
    using in_b = ElemB;
    using acc = Acc;
    using out = Out;
    using math = Math;
    using fp8_policy = Fp8Policy;
    using scale_a = ScaleElemA;
    using scale_b = ScaleElemB;
    static constexpr int vec = Vec;
    static constexpr int scale_vec_a = ScaleVecA;
    static constexpr int scale_vec_b = ScaleVecB;
    static constexpr bool has_scales = !std::is_void_v<ScaleElemA> || !std::is_void_v<ScaleElemB>;
    static constexpr iro::util::u64 id = iro::util::mix_u64(
        iro::util::fnv1a_64_cstr("iro.recipe.precision_ab"),
        iro::util::mix_u64(ElemA::id,
                           iro::util::mix_u64(ElemB::id, iro::util::mix_u64(Acc::id, iro::util::mix_u64(Out::id, Fp8Policy::id)))));
};

}  // namespace iro::recipe

// -------------------------------------------------------------- capabilities ----
namespace iro::cap {

struct sm90 {
    static constexpr int sm_version = 90;
    static constexpr iro::util::u64 id = iro::util::fnv1a_64_cstr("iro.cap.sm90");
    static constexpr bool has_tma = true;
    static constexpr bool has_wgmma = true;
    static constexpr bool has_tcgen05 = false;
    static constexpr int max_smem_bytes = 227 * 1024;
    static constexpr int tmem_columns = 0;
};

// B200.  wgmma.* does not exist on sm_100a: the asynchronous MMA is tcgen05 with
// accumulators in tensor memory (the reference's cap::sm100 still says
// has_wgmma = true, core:3336, which would route to Hopper obligations).
struct sm100 {
    static constexpr int sm_version = 100;
    static constexpr iro::util::u64 id = iro::util::fnv1a_64_cstr("iro.cap.sm100");
    static constexpr bool has_tma = true;
    static constexpr bool has_wgmma = false;
    static constexpr bool has_tcgen05 = true;
    static constexpr int max_smem_bytes = 227 * 1024;
    static constexpr int tmem_columns = 512;
    static constexpr int tmem_lanes = 128;
    static constexpr int max_named_barriers = 16;
    static constexpr int max_regs_per_thread = 255;
    static constexpr int regs_per_sm = 65536;
};

}  // namespace iro::cap

// ------------------------------------------------------- scopes, executors, tokens ----
// The typestate vocabulary of the contracts (reference core: execution groups :763-820, scopes :822-889, token
// families :937-1210, token queries :1458-1650, payload concepts :2566-2590, ports :2949-3010), restated for what the sm100 graphs need: three token
// families (visible_at, alive, sync_at), ordered scopes and lifetimes, and input / output ports that carry them.
namespace iro::scope {
#define IRO_SCOPE(name, lvl)                                                                  \
    struct name {                                                                             \
        static constexpr int level = lvl;                                                     \
        static constexpr iro::util::u64 id = iro::util::fnv1a_64_cstr("iro.scope." #name);    \
    }
IRO_SCOPE(lane, 0);
IRO_SCOPE(warp, 1);
IRO_SCOPE(warpgroup, 2);
IRO_SCOPE(block, 3);
IRO_SCOPE(cluster, 4);
IRO_SCOPE(device, 5);
#undef IRO_SCOPE
}  // namespace iro::scope

namespace iro::exec {
// Who executes an obligation; `scope` is the smallest scope that contains all of its threads.
#define IRO_EXEC(name, scope_name)                                                            \
    struct name {                                                                             \
        using scope = iro::scope::scope_name;                                                 \
        static constexpr iro::util::u64 id = iro::util::fnv1a_64_cstr("iro.exec." #name);     \
    }
IRO_EXEC(lane, lane);              // one elected thread (TMA issue, tcgen05.mma, tcgen05.commit)
IRO_EXEC(warp, warp);
IRO_EXEC(warpgroup, warpgroup);
IRO_EXEC(block, block);
IRO_EXEC(cta_group1, block);       // tensor-core work of one CTA
IRO_EXEC(cta_group2, cluster);     // tensor-core work of a CTA pair
IRO_EXEC(host, device);
#undef IRO_EXEC
}  // namespace iro::exec

namespace iro::scope {
template <class Exec>
using min_scope_for_t = typename Exec::scope;
}  // namespace iro::scope

namespace iro::token {

struct kind_visible_at { static constexpr auto id = iro::util::fnv1a_64_cstr("iro.token.kind_visible_at"); };
struct kind_alive { static constexpr auto id = iro::util::fnv1a_64_cstr("iro.token.kind_alive"); };
struct kind_sync_at { static constexpr auto id = iro::util::fnv1a_64_cstr("iro.token.kind_sync_at"); };

namespace lifetime {
#define IRO_LIFETIME(name, lvl)                                                                 \
    struct name {                                                                               \
        static constexpr int level = lvl;                                                       \
        static constexpr iro::util::u64 id = iro::util::fnv1a_64_cstr("iro.lifetime." #name);   \
    }
IRO_LIFETIME(instruction, 0);
IRO_LIFETIME(warp, 1);
IRO_LIFETIME(warpgroup, 2);
IRO_LIFETIME(block, 3);
IRO_LIFETIME(cluster, 4);
IRO_LIFETIME(kernel, 5);
#undef IRO_LIFETIME
}  // namespace lifetime

// The subject's contents can be read by every thread of `Scope` (and, for async-proxy consumers, by the units that act
// for them).
template <class Subject, class Scope>
struct visible_at {
    using kind = kind_visible_at;
    using subject = Subject;
    using scope = Scope;
    static constexpr int level = Scope::level;
    static constexpr iro::util::u64 id =
        iro::util::mix_u64(iro::util::fnv1a_64_cstr("iro.token.visible_at"), iro::util::mix_u64(Subject::id, Scope::id));
};
// The subject's storage stays allocated for `Lifetime`.
template <class Subject, class Lifetime>
struct alive {
    using kind = kind_alive;
    using subject = Subject;
    using lifetime = Lifetime;
    static constexpr int level = Lifetime::level;
    static constexpr iro::util::u64 id =
        iro::util::mix_u64(iro::util::fnv1a_64_cstr("iro.token.alive"), iro::util::mix_u64(Subject::id, Lifetime::id));
};
// A synchronisation of `Scope` (barrier, mbarrier phase, commit) orders the producer of the subject before its readers.
template <class Subject, class Scope>
struct sync_at {
    using kind = kind_sync_at;
    using subject = Subject;
    using scope = Scope;
    static constexpr int level = Scope::level;
    static constexpr iro::util::u64 id =
        iro::util::mix_u64(iro::util::fnv1a_64_cstr("iro.token.sync_at"), iro::util::mix_u64(Subject::id, Scope::id));
};

}  // namespace iro::token

namespace iro::verify {

// Does `Tokens` hold a token of this kind for this subject (any scope / lifetime)?
template <class Tokens, class Kind, class Subject>
struct has_token_kind_subject_impl;
template <class Kind, class Subject, class... Ts>
struct has_token_kind_subject_impl<iro::util::type_list<Ts...>, Kind, Subject>
    : std::bool_constant<((std::is_same_v<typename Ts::kind, Kind> && std::is_same_v<typename Ts::subject, Subject>) || ...)> {};
template <class Tokens, class Kind, class Subject>
constexpr bool has_token_kind_subject() {
    return has_token_kind_subject_impl<Tokens, Kind, Subject>::value;
}

// Does `Provided` satisfy the token `Need`: same kind and subject, at a scope / lifetime at least as wide?
template <class Provided, class Need>
struct satisfies_impl;
template <class Need, class... Ts>
struct satisfies_impl<iro::util::type_list<Ts...>, Need>
    : std::bool_constant<((std::is_same_v<typename Ts::kind, typename Need::kind> &&
                           std::is_same_v<typename Ts::subject, typename Need::subject> && Ts::level >= Need::level) || ...)> {};
template <class Provided, class Need>
inline constexpr bool satisfies_v = satisfies_impl<Provided, Need>::value;

}  // namespace iro::verify

// ------------------------------------------------- obligations / realizations ----
namespace iro::contract {

// What a port carries (reference core: payload concepts :2566-2590).
namespace space {
struct global { static constexpr auto id = iro::util::fnv1a_64_cstr("iro.space.global"); };
struct shared { static constexpr auto id = iro::util::fnv1a_64_cstr("iro.space.shared"); };
struct tmem { static constexpr auto id = iro::util::fnv1a_64_cstr("iro.space.tmem"); };
struct reg { static constexpr auto id = iro::util::fnv1a_64_cstr("iro.space.reg"); };
}  // namespace space
struct tile_kind {};
struct handle_kind {};
struct scalar_kind {};
// A tile of data in a memory space.
template <class Space>
struct Tile {
    using payload_kind = tile_kind;
    using space = Space;
};
// An opaque handle: tensor map, mbarrier, tensor-memory base address, matrix descriptor.
struct Handle { using payload_kind = handle_kind; };
// A per-thread or per-call value (scales alpha / beta, softmax state).
struct Scalar { using payload_kind = scalar_kind; };
template <class P>
concept TilePayload = std::is_same_v<typename P::payload_kind, tile_kind>;
template <class P>
concept HandlePayload = std::is_same_v<typename P::payload_kind, handle_kind>;

// Ports: what an obligation needs to hold before it runs (`required`) and what holds after it (`provided`).
template <class Payload, class Subject, class ExecGroup, class Required>
struct InputPort {
    static constexpr bool is_input = true;
    using payload = Payload;
    using subject = Subject;
    using exec_group = ExecGroup;
    using required = Required;
};
template <class Payload, class Subject, class ExecGroup, class Provided>
struct OutputPort {
    static constexpr bool is_input = false;
    using payload = Payload;
    using subject = Subject;
    using exec_group = ExecGroup;
    using provided = Provided;
};

namespace subject {
struct global { static constexpr iro::util::u64 id = iro::util::fnv1a_64_cstr("iro.subject.global"); };
}  // namespace subject

// Resources an obligation holds while it runs.
template <int SmemBytes = 0, int TmemCols = 0, int Mbarriers = 0>
struct Resources {
    static constexpr int smem_bytes = SmemBytes;
    static constexpr int tmem_cols = TmemCols;
    static constexpr int mbarriers = Mbarriers;
};

// Base of every obligation: a stable id plus the resources it needs.
template <iro::util::u64 Id, class Res = Resources<>>
struct Obligation {
    static constexpr iro::util::u64 id = Id;
    using resources = Res;
    // Ports; an obligation that moves or makes data overrides them.
    using inputs = iro::util::type_list<>;
    using outputs = iro::util::type_list<>;
};

// Base of every realization (reference core:3290-3300): the id mixes the obligation's id with the implementation id,
// so that one implementation name registered for two obligations yields two realization ids.
template <class ObligationT, iro::util::u64 ImplId>
struct Realization {
    using obligation = ObligationT;
    static constexpr iro::util::u64 impl_id = ImplId;
    static constexpr iro::util::u64 id =
        iro::util::mix_u64(iro::util::fnv1a_64_cstr("iro.contract.Realization"), iro::util::mix_u64(ObligationT::id, ImplId));
};

}  // namespace iro::contract

namespace iro::bind {

template <class RealizationT, class RequiredCap>
struct RealizationEntry {
    using realization = RealizationT;
    using cap = RequiredCap;
};

template <class ObligationT, class RealizationT>
struct Resolved {
    using obligation = ObligationT;
    using realization = RealizationT;
    static constexpr bool found = true;
};

// First entry of `Registry` whose capability the target satisfies
// (Cap::sm_version >= Required::sm_version, reference core:3927-3943).
template <class ObligationT, class Cap, class Registry>
struct lookup_realization;
template <class ObligationT, class Cap>
struct lookup_realization<ObligationT, Cap, iro::util::type_list<>> {
    static_assert(sizeof(ObligationT) == 0, "no realization registered for this obligation on this capability");
};
template <class ObligationT, class Cap, class E, class... Es>
struct lookup_realization<ObligationT, Cap, iro::util::type_list<E, Es...>> {
    using type = std::conditional_t<(Cap::sm_version >= E::cap::sm_version),
                                    Resolved<ObligationT, typename E::realization>,
                                    typename lookup_realization<ObligationT, Cap, iro::util::type_list<Es...>>::type>;
};
template <class ObligationT, class Cap, class E>
struct lookup_realization<ObligationT, Cap, iro::util::type_list<E>> {
    static_assert(Cap::sm_version >= E::cap::sm_version, "no realization for this capability");
    using type = Resolved<ObligationT, typename E::realization>;
};
template <class ObligationT, class Cap, class Registry>
using lookup_realization_t = typename lookup_realization<ObligationT, Cap, Registry>::type;

}  // namespace iro::bind

// ---------------------------------------------------------------- composition ----
namespace iro::compose {

template <class List>
struct sum_resources;
template <class... Os>
struct sum_resources<iro::util::type_list<Os...>> {
    static constexpr int smem_bytes = (0 + ... + Os::resources::smem_bytes);
    static constexpr int tmem_cols = (0 + ... + Os::resources::tmem_cols);
    static constexpr int mbarriers = (0 + ... + Os::resources::mbarriers);
};

// An obligation list checked against the capability's budgets (the reference
// checks smem, named barriers and registers, core:3823-3846; tensor memory is
// added here because sm100 accumulators live there).
template <class Obligations, class Cap, int Threads, int MaxRegsPerThread>
struct Composition {
    using obligations = Obligations;
    using cap = Cap;
    using totals = sum_resources<Obligations>;
    static constexpr int smem_bytes = totals::smem_bytes;
    static constexpr int tmem_cols = totals::tmem_cols;
    static constexpr int mbarriers = totals::mbarriers;
    static constexpr int threads = Threads;
    static_assert(smem_bytes <= Cap::max_smem_bytes, "composition exceeds the shared-memory budget");
    static_assert(tmem_cols <= Cap::tmem_columns, "composition exceeds the tensor-memory columns");
    static_assert(MaxRegsPerThread <= Cap::max_regs_per_thread, "register budget above the per-thread limit");
    static_assert(Threads % 128 == 0, "warpgroup roles need a multiple of 128 threads");
    static constexpr iro::util::u64 id = iro::util::hash_list<Obligations>::value;
};

}  // namespace iro::compose
