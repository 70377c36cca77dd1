// Subjects = (tag, index) wires (reference include/axp/naming/subjects.hpp:7-52).
#pragma once
#include "tags.hpp"

namespace axp::subject {

using global = iro::contract::subject::global;

template <class Tag, int I>
struct wire {
    using tag = Tag;
    static constexpr int index = I;
    static constexpr auto id = iro::util::mix_u64(Tag::id, static_cast<iro::util::u64>(I));
};

using MatrixA = wire<axp::tag::A, 0>;
using MatrixB = wire<axp::tag::B, 0>;
using MatrixC = wire<axp::tag::C, 0>;
using Accumulator = wire<axp::tag::Acc, 0>;
using Output = wire<axp::tag::O, 0>;
using AttentionQ = wire<axp::tag::Q, 0>;
using AttentionK = wire<axp::tag::K, 0>;
using AttentionV = wire<axp::tag::V, 0>;
using AttentionS = wire<axp::tag::S, 0>;
using AttentionP = wire<axp::tag::P, 0>;
using ScaleA = wire<axp::tag::ScaleA, 0>;
using ScaleB = wire<axp::tag::ScaleB, 0>;

using SoftmaxState = wire<axp::tag::State, 0>;

// A subject in a memory space: the token subject of "the A tile as it sits in shared memory", "the accumulator in tensor
// memory", "the scores in registers".  Moving data between spaces is what the data-movement obligations do, so their
// input and output ports name the same wire in two spaces.
template <class Space, class Subj>
struct at {
    using space = Space;
    using base = Subj;
    static constexpr auto id = iro::util::mix_u64(iro::util::mix_u64(iro::util::fnv1a_64_cstr("axp.subject.at"), Space::id), Subj::id);
};
template <class Subj>
using in_global = at<iro::contract::space::global, Subj>;
template <class Subj>
using in_shared = at<iro::contract::space::shared, Subj>;
template <class Subj>
using in_tmem = at<iro::contract::space::tmem, Subj>;
template <class Subj>
using in_regs = at<iro::contract::space::reg, Subj>;

// Handles: the tensor map that describes a global tensor, and the base address of a tensor-memory allocation.
template <class Subj>
struct tensor_map_of {
    using base = Subj;
    static constexpr auto id = iro::util::mix_u64(iro::util::fnv1a_64_cstr("axp.subject.tensor_map_of"), Subj::id);
};
struct tmem_base {
    static constexpr auto id = iro::util::fnv1a_64_cstr("axp.subject.tmem_base");
};

template <class T>
struct is_subject : std::false_type {};
template <class Tag, int I>
struct is_subject<wire<Tag, I>> : std::true_type {};
template <>
struct is_subject<global> : std::true_type {};
template <class Space, class Subj>
struct is_subject<at<Space, Subj>> : std::true_type {};

}  // namespace axp::subject
