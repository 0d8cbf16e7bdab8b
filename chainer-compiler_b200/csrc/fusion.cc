// Compile-time (host) pieces that decide what the kernels see: which nodes form a fused
// elementwise group, and how fp32 weights become int8/uint8.
#include <math.h>
#include <string.h>

#include <set>
#include <stack>
#include <string>
#include <vector>

#include "common.h"

namespace chxq {
namespace {

bool is_float_or_unknown(int dtype) {
    return dtype == 0 || dtype == CHXQ_FLOAT16 || dtype == CHXQ_FLOAT32 || dtype == CHXQ_FLOAT64;
}

// Node::IsZeroCost (compiler/node.cc:249-252).
bool is_zero_cost(const std::string& op) {
    return op == "Identity" || op == "Constant" || op == "Reshape";
}

}  // namespace
}  // namespace chxq

using namespace chxq;

// FuseElementwiseOperations (compiler/fusion_elementwise.cc:10-40) decides what is fusable;
// FuseAllConnectedNodes (compiler/fusion.cc:165-214) floods over producer/user edges, then drops
// members that would close a cycle through a non-member (RejectCyclicNodes, :26-58) and constants no
// member reads (RejectUnusedConstants, :60-79); a group needs at least two nodes that are not
// Identity/Constant/Reshape.  Group ids are handed out in node order, 1-based.
// One difference: a node that already belongs to a group is not entered again by a later flood (the
// reference CHECK-fails there, compiler/fusion.cc:178).
extern "C" int chxq_fuse_elementwise(
        const chxq_graph_node* nodes, int32_t n_nodes, const chxq_graph_value* values, int32_t n_values, int32_t* group_of_node,
        int32_t* n_groups) {
    CHXQ_CHECK_ARG(nodes && values && group_of_node && n_nodes >= 0 && n_values >= 0, "fuse_elementwise: null argument");
    static const std::set<std::string> kFusable = {"Identity", "Add", "Sub", "Mul", "Tanh", "Sigmoid", "Exp"};
    std::vector<int> producer(n_values, -1);
    std::vector<std::vector<int>> users(n_values);
    for (int i = 0; i < n_nodes; ++i) {
        CHXQ_CHECK_ARG(nodes[i].op_type != nullptr, "fuse_elementwise: node %d has no op type", i);
        for (int k = 0; k < nodes[i].n_inputs; ++k) {
            const int v = nodes[i].inputs[k];
            if (v < 0) continue;  // absent optional input
            CHXQ_CHECK_ARG(v < n_values, "fuse_elementwise: node %d reads value %d out of range", i, v);
            users[v].push_back(i);
        }
        for (int k = 0; k < nodes[i].n_outputs; ++k) {
            const int v = nodes[i].outputs[k];
            CHXQ_CHECK_ARG(v >= 0 && v < n_values, "fuse_elementwise: node %d writes value %d out of range", i, v);
            producer[v] = i;
        }
    }
    auto fusable = [&](int i) {
        const chxq_graph_node& nd = nodes[i];
        const std::string op = nd.op_type;
        if (op == "Constant") return nd.const_is_float != 0 && nd.const_num_elements == 1;
        if (!kFusable.count(op)) return false;
        for (int k = 0; k < nd.n_inputs; ++k) {
            const int v = nd.inputs[k];
            if (v >= 0 && !is_float_or_unknown(values[v].dtype)) return false;
        }
        return true;
    };

    std::vector<int> group(n_nodes, 0);
    int num_groups = 0;
    for (int base = 0; base < n_nodes; ++base) {
        if (group[base] != 0 || !fusable(base)) continue;
        std::set<int> cands;
        std::stack<int> st;
        st.push(base);
        while (!st.empty()) {
            const int nd = st.top();
            st.pop();
            if (group[nd] != 0) continue;
            if (!cands.insert(nd).second) continue;
            for (int k = 0; k < nodes[nd].n_inputs; ++k) {
                const int v = nodes[nd].inputs[k];
                if (v < 0) continue;
                const int p = producer[v];
                if (p < 0 || !fusable(p) || nodes[p].is_grad != nodes[base].is_grad) continue;
                st.push(p);
            }
            for (int k = 0; k < nodes[nd].n_outputs; ++k) {
                for (int u : users[nodes[nd].outputs[k]]) {
                    if (!fusable(u) || nodes[u].is_grad != nodes[base].is_grad) continue;
                    st.push(u);
                }
            }
        }
        // RejectCyclicNodes: walk downstream from every non-member that reads a member's output; any
        // member reached that way depends on the group through the outside and must leave.
        {
            std::stack<int> q;
            for (int nd : cands)
                for (int k = 0; k < nodes[nd].n_outputs; ++k)
                    for (int u : users[nodes[nd].outputs[k]])
                        if (!cands.count(u)) q.push(u);
            std::set<int> seen, rejected;
            while (!q.empty()) {
                const int nd = q.top();
                q.pop();
                if (!seen.insert(nd).second) continue;
                if (cands.count(nd)) rejected.insert(nd);
                for (int k = 0; k < nodes[nd].n_outputs; ++k)
                    for (int u : users[nodes[nd].outputs[k]]) q.push(u);
            }
            for (int nd : rejected) cands.erase(nd);
        }
        // RejectUnusedConstants.
        {
            std::set<int> rejected;
            for (int nd : cands) {
                if (strcmp(nodes[nd].op_type, "Constant") != 0) continue;
                bool used = false;
                for (int u : users[nodes[nd].outputs[0]]) used = used || cands.count(u) > 0;
                if (!used) rejected.insert(nd);
            }
            for (int nd : rejected) cands.erase(nd);
        }
        int num_calc = 0;
        for (int nd : cands) num_calc += !is_zero_cost(nodes[nd].op_type);
        if (num_calc < 2) continue;
        ++num_groups;
        for (int nd : cands) group[nd] = num_groups;
    }
    memcpy(group_of_node, group.data(), sizeof(int32_t) * (size_t)n_nodes);
    if (n_groups) *n_groups = num_groups;
    return CHXQ_OK;
}

// QuantizeData (compiler/quantize.cc:70-89).
static void quantize_block(const float* w, int64_t n, bool to_int8, void* q, float* scale_out, int32_t* zp_out) {
    float rmin = 0.f, rmax = 0.f;  // :71-72 the range always includes zero
    for (int64_t i = 0; i < n; ++i) {
        rmin = w[i] < rmin ? w[i] : rmin;
        rmax = w[i] > rmax ? w[i] : rmax;
    }
    if (to_int8) {
        const float max_range = fmaxf(fabsf(rmin), fabsf(rmax));
        const float scale = max_range * 2 / 254.f;
        int8_t* out = static_cast<int8_t*>(q);
        // SlowRound (runtime/chainerx_util.cc:397-410): fp32 quotient, rint in double, back to fp32, then AsType.
        for (int64_t i = 0; i < n; ++i) out[i] = static_cast<int8_t>(static_cast<int32_t>(static_cast<float>(rint(static_cast<double>(w[i] / scale)))));
        *scale_out = scale;
        *zp_out = 0;
    } else {
        const float scale = rmin != rmax ? (rmax - rmin) / 255.f : 1.f;
        const int64_t zp = static_cast<int64_t>(rint(static_cast<double>((0 - rmin) / scale)));
        uint8_t* out = static_cast<uint8_t*>(q);
        for (int64_t i = 0; i < n; ++i) {
            const float v = static_cast<float>(rint(static_cast<double>(w[i] / scale))) + static_cast<float>(zp);
            out[i] = static_cast<uint8_t>(static_cast<int32_t>(v));  // low eight bits of the truncated integer
        }
        *scale_out = scale;
        *zp_out = static_cast<int32_t>(zp);
    }
}

extern "C" int chxq_quantize_weights_host(
        const float* w, int64_t M, int64_t inner, int32_t to_int8, int32_t per_channel, void* q, float* scales, int32_t* zero_points) {
    CHXQ_CHECK_ARG(w && q && scales && zero_points && M > 0 && inner > 0, "quantize_weights: bad arguments");
    if (!per_channel) {
        quantize_block(w, M * inner, to_int8 != 0, q, scales, zero_points);
        return CHXQ_OK;
    }
    // QuantizeWeightConvolution (compiler/quantize.cc:98-129): one QuantizeData per output channel.
    for (int64_t m = 0; m < M; ++m)
        quantize_block(w + m * inner, inner, to_int8 != 0, static_cast<char*>(q) + m * inner, scales + m, zero_points + m);
    return CHXQ_OK;
}
