// Order in which a network's parameterised layers finish their backward pass, containers included.
//
// cuTAGI's own DDPSequential::sync_parameters walks `model->layers` only (src/ddp.cpp:113-146), so the Conv2d and
// BatchNorm2d layers inside LayerBlock / ResNetBlock containers are never exchanged. The walk below descends into the
// containers and visits the leaves in the order the backward pass reaches them: layers last to first
// (src/sequential.cpp:392-410), a LayerBlock's layers last to first (src/layer_block.cpp:196-219), a residual block's
// main block before its shortcut (src/resnet_block.cpp:244-277). That is the order in which parameter deltas become
// available, which is the order the exchange wants its buckets filled in.
//
// The walk itself knows nothing about cuTAGI's classes: `children(node, out)` appends a container's children in FORWARD
// order (for a residual block: main block, then shortcut) and returns true, or returns false for a leaf; `visit(leaf)` is
// called for every leaf. ddp_b200.cpp supplies the two for cuTAGI's BaseLayer tree.
#pragma once
#include <vector>

template <class Node, class Children, class Visit>
void ddp_b200_walk_backward(const std::vector<Node> &forward_order, Children &&children, Visit &&visit) {
    for (auto it = forward_order.rbegin(); it != forward_order.rend(); ++it) {
        std::vector<Node> kids;
        int kind = children(*it, kids);  // 0: leaf, 1: sequence (reversed in backward), 2: residual block (main, shortcut)
        if (kind == 0) {
            visit(*it);
        } else if (kind == 1) {
            ddp_b200_walk_backward(kids, children, visit);
        } else {
            // main block first, then the shortcut: each is one node whose own children are walked in reverse
            for (auto &k : kids) ddp_b200_walk_backward(std::vector<Node>{k}, children, visit);
        }
    }
}
