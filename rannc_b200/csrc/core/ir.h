// Graph IR: types, values, nodes, graphs, and their msgpack layout.
//
// The IR mirrors what the reference keeps per traced model
// (src/graph/ir.h:25-615): a bipartite graph of operator nodes and named
// values, where a value is a tensor / scalar / list / tuple with a static
// shape, flagged as parameter, batch-dependent or loss.  Field order of the
// serialised form follows the reference so deployment files stay readable:
//   IRType  : base_type, scalar_type, tensor_dim, tensor_elem_type, requires_grad,
//             list_type, compound_types, list_size, func_name      (ir.h:225-227)
//   IRValue : name, type, is_param, is_batch, is_loss, batch_size   (ir.h:381)
//   IRNode  : name, input_names, output_names, id, is_criterion, is_batch,
//             batch_size                                            (ir.h:458-459)
//   IRGraph : name, nodes, values, input_names, output_names, is_replicable,
//             batch_size                                            (ir.h:603-604)
// The IR here is filled from a torch.export / FX graph instead of a
// TorchScript trace; operator names use the "aten::linear" spelling.
#pragma once
#include <cstdint>
#include <map>
#include <set>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "msgpack.h"

namespace rannc {

enum class IRBaseType : int { SCALAR = 0, TENSOR, STRING, LIST, TUPLE, OPTIONAL, NONE, FUNCTION };
enum class IRTensorElemType : int { UNDEF = 0, INT, DOUBLE, FLOAT, HALF, BFLOAT16, LONG, BOOL };
enum class IRListType : int { INT = 0, FLOAT, BOOL, TENSOR, GENERIC };
enum class IRScalarType : int { NONE = 0, INT, FLOAT, NUMBER, BOOL, DEVICE };

size_t elemSize(IRTensorElemType t);
const char* elemTypeName(IRTensorElemType t);

struct IRType {
    IRBaseType base_type = IRBaseType::NONE;
    IRScalarType scalar_type = IRScalarType::NONE;
    std::vector<int64_t> tensor_dim;
    IRTensorElemType tensor_elem_type = IRTensorElemType::UNDEF;
    bool requires_grad = false;
    IRListType list_type = IRListType::GENERIC;
    std::vector<IRType> compound_types;
    uint64_t list_size = static_cast<uint64_t>(-1);
    std::string func_name;

    static IRType tensor(IRTensorElemType elem, std::vector<int64_t> dims, bool requires_grad = false);
    static IRType scalar(IRScalarType st);
    static IRType list(IRListType lt, std::vector<IRType> elems);
    static IRType tuple(std::vector<IRType> elems);
    static IRType none();
    static IRType string();

    int64_t numel() const;     // tensors: product of dims; compound: sum over elements
    int64_t sizeInByte() const;
    // scale dim 0 of every tensor inside: new = dim0 * num / den (reference: ir.cpp:211-237)
    void scaleBatch(int64_t num, int64_t den);
    bool holdsGradient() const;  // float tensor types (reference: src/Common.cpp:80-146)

    mp::Value pack() const;
    static IRType unpack(const mp::Value& v);
};

struct IRValue {
    std::string name;
    IRType type;
    bool is_param = false;
    bool is_batch = false;
    bool is_loss = false;
    int64_t batch_size = 0;
    // not serialised: extra axis a later sequence/context split could use
    int split_dim = 0;
    // not serialised: what the tracer knows about the first dimension from symbolic shapes.  +1: it is the
    // (symbolic) batch, -1: the tensor has no batch-sized dimension at all (a reduction over the batch, a
    // statistic), 0: unknown, the classifier's propagation rule decides.
    int batch_hint = 0;

    mp::Value pack() const;
    static IRValue unpack(const mp::Value& v);
};

struct IRNode {
    std::string name;  // operator, e.g. "aten::linear"
    std::vector<std::string> input_names;
    std::vector<std::string> output_names;
    std::string id;  // unique node id (the FX node name)
    bool is_criterion = false;
    bool is_batch = false;
    int64_t batch_size = 0;

    mp::Value pack() const;
    static IRNode unpack(const mp::Value& v);
};

struct IRGraph {
    std::string name;
    std::vector<IRNode> nodes;  // topological order
    std::unordered_map<std::string, IRValue> values;
    std::vector<std::string> input_names;   // real inputs first, then params/buffers
    std::vector<std::string> output_names;
    bool is_replicable = true;
    int64_t batch_size = 0;

    const IRValue& value(const std::string& n) const;
    IRValue& value(const std::string& n);
    bool hasValue(const std::string& n) const { return values.count(n) != 0; }
    bool isInput(const std::string& n) const;

    std::vector<std::string> paramInputNames() const;
    std::vector<std::string> nonParamInputNames() const;
    int64_t paramSizeInByte() const;
    int64_t inputSizeInByte() const;   // non-parameter inputs
    int64_t outputSizeInByte() const;

    // inputs + outputs + input gradients + 2 x shared-input clones (reference: ir.cpp:852-897)
    int64_t commBufSize() const;

    void check() const;  // every node input defined before use; outputs unique
    mp::Value pack() const;
    static IRGraph unpack(const mp::Value& v);
    std::string toString() const;
    std::string toDot() const;
};

// name -> nodes that read the value / the node that writes it
std::unordered_map<std::string, std::vector<size_t>> consumers(const IRGraph& g);
std::unordered_map<std::string, size_t> producers(const IRGraph& g);

// Values that no node and no graph output uses (reference: ir.cpp:702-760).
std::vector<std::string> findUnusedValues(const IRGraph& g);
// Drops nodes whose outputs reach no graph output (reference: ir.cpp:762-850).
IRGraph removeUnusedNodes(const IRGraph& g);
// Returns a copy scaled to a different batch size: dim 0 of every batch value is
// multiplied by new_bs / g.batch_size (reference: Decomposition.cpp:943-1008).
IRGraph scaleGraph(const IRGraph& g, int64_t new_bs);
// Names of inputs that more than one node reads (cloned per use, gradients
// summed, in the stage executor; reference: ir.cpp:537-617).
std::vector<std::string> sharedInputs(const IRGraph& g);

// Labels BATCH / PARAM / CONST / LOSS values and nodes in topological order
// (reference: src/graph/GuessValueTypes.cpp:50-263).
void guessValueTypes(IRGraph& g);

// Path into a nested list / tuple value (reference: src/torch/IValueLocation.h:16-62).
struct StepInIValue {
    int type = 0;  // 0 LIST, 1 TUPLE
    int64_t index = 0;
};
struct IValueLocation {
    std::string value_name;
    std::vector<StepInIValue> path;
    mp::Value pack() const;
    static IValueLocation unpack(const mp::Value& v);
    std::string toString() const;
    bool operator==(const IValueLocation& o) const;
};

// helpers shared by the serialisers
mp::Value packStrings(const std::vector<std::string>& v);
std::vector<std::string> unpackStrings(const mp::Value& v);
mp::Value packInts(const std::vector<int64_t>& v);
std::vector<int64_t> unpackInts(const mp::Value& v);

}  // namespace rannc
