// Structured row addressing of node tensors (node, component, channel) for the linears.
#pragma once

namespace sxb {

// Logical row g: node = first_node + g / components, m = g % components,
// address = node*node_stride + offset + m*component_stride (in elements).
struct RowMap {
    long node_stride;
    long component_stride;
    long offset;
    int components;
};

}  // namespace sxb
