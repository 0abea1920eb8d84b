// Shape/stride algebra for device tensors.  Strides are in elements and may be zero (broadcast)
// or negative (flip).  Same operations and flags as the reference's `StridedShape`
// (kn-cuda-eval/src/shape.rs:11-344); `view` follows the contiguous-group rule documented there.
#pragma once
#include <optional>
#include <string>
#include <vector>

#include "common.h"

namespace kn {

struct StridedShape {
    std::vector<int64_t> shape;
    std::vector<int64_t> strides;

    StridedShape() = default;
    StridedShape(std::vector<int64_t> shape_, std::vector<int64_t> strides_);
    static StridedShape simple(const std::vector<int64_t>& shape);

    int rank() const { return (int)shape.size(); }
    int64_t size() const;
    bool has_simple_strides() const;   // equal to the row-major strides of `shape`
    bool has_dense_strides() const;    // covers its data range exactly once (any axis order / sign)

    StridedShape slice(int axis, int64_t start, int64_t end, int64_t step) const;
    StridedShape flip(int axis) const;
    StridedShape broadcast(const std::vector<int64_t>& new_shape) const;
    StridedShape permute(const std::vector<int>& permutation) const;
    std::optional<StridedShape> view(const std::vector<int64_t>& new_shape) const;

    // lowest and highest element offset reachable (both 0 for empty shapes)
    void extent(int64_t* lo, int64_t* hi) const;
    std::string str() const;
    bool operator==(const StridedShape& o) const { return shape == o.shape && strides == o.strides; }
};

std::vector<int64_t> simple_strides(const std::vector<int64_t>& shape);

}  // namespace kn
