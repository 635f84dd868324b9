// pkg_ext.h -- EXTENSION to the builder rungs: NOT part of the reference's pkg surface.
//
// The reference's rungs admit a store only after a reduction (pkg/chain.go:433-438: MidChain has no Store;
// "v0 pkg rungs require at least one reduction before the store"), so a rank-preserving map -- the last
// statement of a softmax or a layer-norm, a bias add, an activation -- cannot be stored through them. The
// kernel library has that operator (tcab_map), and a chain written statement by statement needs it for its
// last step. This file adds the one missing rung, kept apart from pkg.h so that everything in pkg.h stays a
// mirror of the reference:
//
//     Iter(..).Map(ops, f).As(..) --ext::StoreMap(t, axes)--> stored
//
// with the same checks as the reference's store (declared tensor, positional axes, live axes only) and the
// additional requirement that the stored axes are all the live axes, in order (a map cannot drop an axis).
#pragma once

#include "pkg.h"

namespace tcab {
namespace pkg {
namespace ext {

Result<Stored> StoreMap(MidChain mid, const Tensor& t, const std::vector<Dim>& axes);

}  // namespace ext
}  // namespace pkg
}  // namespace tcab
