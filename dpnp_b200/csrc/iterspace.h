// Host-side iteration-space algebra: collapsing of shapes/strides shared by up
// to four arrays, order-preserving compaction, memory-extent and overlap
// tests, and helpers to read dpb_array descriptors.
#pragma once

#include <stdint.h>

#include <vector>

#include "../../include/dpnp_b200.h"

namespace dpb {

constexpr int kMaxArrays = 4;

// Collapsed iteration space of up to four arrays.
struct IterSpace {
    int nd = 0;
    int narrays = 0;
    std::vector<int64_t> shape;                 // nd
    std::vector<int64_t> strides[kMaxArrays];   // nd each
    int64_t offsets[kMaxArrays] = {0, 0, 0, 0}; // element offsets
};

// Collapse in place. `strides` holds narrays*nd values laid out [array][dim].
// Returns the new nd. See dpb_simplify_iteration_space in the public header.
int simplify_iteration_space(int narrays, int nd, int64_t *shape, int64_t *strides,
                             int64_t *offsets);

// Order-preserving merge of neighbouring dimensions; returns the new nd.
int compact_iteration(int nd, int64_t *shape, int64_t *strides);

// Strides of the descriptor as a vector (C-contiguous strides are
// materialised when the descriptor carries none).
std::vector<int64_t> strides_of(const dpb_array &a);
int64_t num_elements(const dpb_array &a);

// Smallest and largest element displacement reachable from `data`.
void displacement_range(const dpb_array &a, int64_t &lo, int64_t &hi);

bool arrays_overlap(const dpb_array &a, const dpb_array &b);
bool same_logical_tensors(const dpb_array &a, const dpb_array &b);

// Validate a descriptor (nd range, pointers, typenum); sets the error message.
int check_array(const dpb_array *a, const char *what);

}  // namespace dpb
