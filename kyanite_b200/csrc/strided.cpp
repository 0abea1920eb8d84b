#include "strided.h"

#include <algorithm>
#include <cstdlib>
#include <numeric>

#include "kn_b200.h"

namespace kn {

std::vector<int64_t> simple_strides(const std::vector<int64_t>& shape) {
    std::vector<int64_t> s(shape.size());
    int64_t next = 1;
    for (int i = (int)shape.size() - 1; i >= 0; i--) {
        s[i] = next;
        next *= shape[i];
    }
    return s;
}

StridedShape::StridedShape(std::vector<int64_t> shape_, std::vector<int64_t> strides_)
    : shape(std::move(shape_)), strides(std::move(strides_)) {
    KN_CHECK(shape.size() == strides.size(), KN_ERR_INTERNAL, "shape and stride rank mismatch");
}

StridedShape StridedShape::simple(const std::vector<int64_t>& shape) { return StridedShape(shape, simple_strides(shape)); }

int64_t StridedShape::size() const {
    int64_t n = 1;
    for (int64_t d : shape) n *= d;
    return n;
}

bool StridedShape::has_simple_strides() const { return strides == simple_strides(shape); }

bool StridedShape::has_dense_strides() const {
    if (size() == 0) return true;
    std::vector<std::pair<int64_t, int64_t>> pairs;   // (|stride|, size)
    for (int i = 0; i < rank(); i++) pairs.push_back({std::llabs(strides[i]), shape[i]});
    std::stable_sort(pairs.begin(), pairs.end(), [](auto& a, auto& b) { return a.first > b.first; });
    std::vector<int64_t> sorted_shape, sorted_strides;
    for (auto& p : pairs) {
        sorted_shape.push_back(p.second);
        sorted_strides.push_back(p.first);
    }
    return simple_strides(sorted_shape) == sorted_strides;
}

StridedShape StridedShape::slice(int axis, int64_t start, int64_t end, int64_t step) const {
    KN_CHECK(axis >= 0 && axis < rank(), KN_ERR_SHAPE, "slice axis out of range");
    KN_CHECK(step >= 1 && end >= start && (end - start) % step == 0, KN_ERR_SHAPE, "invalid slice range");
    KN_CHECK(start == end || (start < shape[axis] && end - (step - 1) <= shape[axis]), KN_ERR_SHAPE,
             "slice range out of bounds");
    StridedShape r = *this;
    r.shape[axis] = (end - start) / step;
    r.strides[axis] *= step;
    return r;
}

StridedShape StridedShape::flip(int axis) const {
    KN_CHECK(axis >= 0 && axis < rank(), KN_ERR_SHAPE, "flip axis out of range");
    StridedShape r = *this;
    r.strides[axis] = -r.strides[axis];
    return r;
}

StridedShape StridedShape::broadcast(const std::vector<int64_t>& new_shape) const {
    KN_CHECK((int)new_shape.size() == rank(), KN_ERR_SHAPE, "broadcast must keep the rank");
    StridedShape r = *this;
    for (int i = 0; i < rank(); i++) {
        if (new_shape[i] != shape[i]) {
            KN_CHECK(shape[i] == 1, KN_ERR_SHAPE, "broadcast of a non-unit axis");
            r.shape[i] = new_shape[i];
            r.strides[i] = 0;
        }
    }
    return r;
}

StridedShape StridedShape::permute(const std::vector<int>& permutation) const {
    KN_CHECK((int)permutation.size() == rank(), KN_ERR_SHAPE, "permutation rank mismatch");
    std::vector<bool> seen(rank(), false);
    StridedShape r;
    for (int p : permutation) {
        KN_CHECK(p >= 0 && p < rank() && !seen[p], KN_ERR_SHAPE, "invalid permutation");
        seen[p] = true;
        r.shape.push_back(shape[p]);
        r.strides.push_back(strides[p]);
    }
    return r;
}

std::optional<StridedShape> StridedShape::view(const std::vector<int64_t>& new_shape) const {
    int64_t new_size = 1;
    for (int64_t d : new_shape) new_size *= d;
    KN_CHECK(new_size == size(), KN_ERR_SHAPE, "view must keep the element count");
    if (size() == 0 || rank() == 0) return StridedShape::simple(new_shape);

    // maximal runs of axes that are contiguous with each other: (element count, stride of last axis)
    std::vector<std::pair<int64_t, int64_t>> groups;
    {
        int64_t group_size = 1;
        bool have_prev = false;
        int64_t prev_stride = 0;
        for (int i = 0; i < rank(); i++) {
            if (have_prev && prev_stride != shape[i] * strides[i]) {
                groups.push_back({group_size, prev_stride});
                group_size = 1;
            }
            group_size *= shape[i];
            prev_stride = strides[i];
            have_prev = true;
        }
        groups.push_back({group_size, prev_stride});
    }

    std::vector<int64_t> new_strides(new_shape.size(), 0);
    size_t next_d = 0;
    for (auto& g : groups) {
        int64_t left = g.first;
        while (left > 1) {
            if (next_d >= new_shape.size()) return std::nullopt;
            int64_t d = new_shape[next_d];
            if (d == 0 || left % d != 0) return std::nullopt;
            left /= d;
            new_strides[next_d] = left * g.second;
            next_d++;
        }
    }
    for (size_t d = next_d; d < new_shape.size(); d++) {
        if (new_shape[d] != 1) return std::nullopt;
        new_strides[d] = 1;
    }
    return StridedShape(new_shape, new_strides);
}

void StridedShape::extent(int64_t* lo, int64_t* hi) const {
    *lo = 0;
    *hi = 0;
    if (size() == 0) return;
    for (int i = 0; i < rank(); i++) {
        int64_t reach = (shape[i] - 1) * strides[i];
        if (reach < 0) *lo += reach; else *hi += reach;
    }
}

std::string StridedShape::str() const {
    std::string s = "[";
    for (int i = 0; i < rank(); i++) s += (i ? "," : "") + std::to_string(shape[i]);
    s += "]/[";
    for (int i = 0; i < rank(); i++) s += (i ? "," : "") + std::to_string(strides[i]);
    return s + "]";
}

}  // namespace kn
