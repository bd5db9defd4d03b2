#include "ir.h"

#include <algorithm>
#include <functional>
#include <sstream>
#include <stdexcept>

namespace rannc {

size_t elemSize(IRTensorElemType t) {
    switch (t) {
        case IRTensorElemType::INT: return 4;
        case IRTensorElemType::DOUBLE: return 8;
        case IRTensorElemType::FLOAT: return 4;
        case IRTensorElemType::HALF: return 2;
        case IRTensorElemType::BFLOAT16: return 2;
        case IRTensorElemType::LONG: return 8;
        case IRTensorElemType::BOOL: return 1;
        default: return 0;
    }
}

const char* elemTypeName(IRTensorElemType t) {
    switch (t) {
        case IRTensorElemType::INT: return "int";
        case IRTensorElemType::DOUBLE: return "double";
        case IRTensorElemType::FLOAT: return "float";
        case IRTensorElemType::HALF: return "half";
        case IRTensorElemType::BFLOAT16: return "bfloat16";
        case IRTensorElemType::LONG: return "long";
        case IRTensorElemType::BOOL: return "bool";
        default: return "undef";
    }
}

// ---------------------------------------------------------------- helpers
mp::Value packStrings(const std::vector<std::string>& v) {
    mp::Array a;
    a.reserve(v.size());
    for (const auto& s : v) a.push_back(mp::Value::str(s));
    return mp::Value::array(std::move(a));
}
std::vector<std::string> unpackStrings(const mp::Value& v) {
    std::vector<std::string> r;
    for (const auto& e : v.as_array()) r.push_back(e.as_str());
    return r;
}
mp::Value packInts(const std::vector<int64_t>& v) {
    mp::Array a;
    a.reserve(v.size());
    for (auto x : v) a.push_back(mp::Value::integer(x));
    return mp::Value::array(std::move(a));
}
std::vector<int64_t> unpackInts(const mp::Value& v) {
    std::vector<int64_t> r;
    for (const auto& e : v.as_array()) r.push_back(e.as_int());
    return r;
}

// ---------------------------------------------------------------- IRType
IRType IRType::tensor(IRTensorElemType elem, std::vector<int64_t> dims, bool rg) {
    IRType t;
    t.base_type = IRBaseType::TENSOR;
    t.tensor_elem_type = elem;
    t.tensor_dim = std::move(dims);
    t.requires_grad = rg;
    return t;
}
IRType IRType::scalar(IRScalarType st) {
    IRType t;
    t.base_type = IRBaseType::SCALAR;
    t.scalar_type = st;
    return t;
}
IRType IRType::list(IRListType lt, std::vector<IRType> elems) {
    IRType t;
    t.base_type = IRBaseType::LIST;
    t.list_type = lt;
    t.list_size = elems.size();
    t.compound_types = std::move(elems);
    return t;
}
IRType IRType::tuple(std::vector<IRType> elems) {
    IRType t;
    t.base_type = IRBaseType::TUPLE;
    t.compound_types = std::move(elems);
    return t;
}
IRType IRType::none() { return IRType(); }
IRType IRType::string() {
    IRType t;
    t.base_type = IRBaseType::STRING;
    return t;
}

int64_t IRType::numel() const {
    if (base_type == IRBaseType::TENSOR) {
        int64_t n = 1;
        for (auto d : tensor_dim) n *= d;
        return n;
    }
    int64_t n = 0;
    for (const auto& c : compound_types) n += c.numel();
    return n;
}

int64_t IRType::sizeInByte() const {
    if (base_type == IRBaseType::TENSOR) return numel() * static_cast<int64_t>(elemSize(tensor_elem_type));
    if (base_type == IRBaseType::SCALAR) return 8;
    int64_t n = 0;
    for (const auto& c : compound_types) n += c.sizeInByte();
    return n;
}

void IRType::scaleBatch(int64_t num, int64_t den) {
    if (base_type == IRBaseType::TENSOR) {
        if (!tensor_dim.empty() && den > 0) {
            // ceil so that a value is never planned smaller than it can be at run time
            tensor_dim[0] = (tensor_dim[0] * num + den - 1) / den;
            if (tensor_dim[0] < 1) tensor_dim[0] = 1;
        }
        return;
    }
    for (auto& c : compound_types) c.scaleBatch(num, den);
}

bool IRType::holdsGradient() const {
    if (base_type == IRBaseType::TENSOR)
        return tensor_elem_type == IRTensorElemType::FLOAT || tensor_elem_type == IRTensorElemType::HALF ||
               tensor_elem_type == IRTensorElemType::BFLOAT16 || tensor_elem_type == IRTensorElemType::DOUBLE;
    for (const auto& c : compound_types)
        if (c.holdsGradient()) return true;
    return false;
}

mp::Value IRType::pack() const {
    mp::Array comp;
    for (const auto& c : compound_types) comp.push_back(c.pack());
    return mp::Value::array({mp::Value::integer(static_cast<int>(base_type)),
                             mp::Value::integer(static_cast<int>(scalar_type)), packInts(tensor_dim),
                             mp::Value::integer(static_cast<int>(tensor_elem_type)),
                             mp::Value::boolean(requires_grad),
                             mp::Value::integer(static_cast<int>(list_type)), mp::Value::array(std::move(comp)),
                             mp::Value::uinteger(list_size), mp::Value::str(func_name)});
}

IRType IRType::unpack(const mp::Value& v) {
    IRType t;
    t.base_type = static_cast<IRBaseType>(v.at(0).as_int());
    t.scalar_type = static_cast<IRScalarType>(v.at(1).as_int());
    t.tensor_dim = unpackInts(v.at(2));
    t.tensor_elem_type = static_cast<IRTensorElemType>(v.at(3).as_int());
    t.requires_grad = v.at(4).as_bool();
    t.list_type = static_cast<IRListType>(v.at(5).as_int());
    for (const auto& c : v.at(6).as_array()) t.compound_types.push_back(IRType::unpack(c));
    t.list_size = v.at(7).as_uint();
    t.func_name = v.at(8).as_str();
    return t;
}

// ---------------------------------------------------------------- IRValue / IRNode
mp::Value IRValue::pack() const {
    return mp::Value::array({mp::Value::str(name), type.pack(), mp::Value::boolean(is_param),
                             mp::Value::boolean(is_batch), mp::Value::boolean(is_loss),
                             mp::Value::integer(batch_size)});
}
IRValue IRValue::unpack(const mp::Value& v) {
    IRValue r;
    r.name = v.at(0).as_str();
    r.type = IRType::unpack(v.at(1));
    r.is_param = v.at(2).as_bool();
    r.is_batch = v.at(3).as_bool();
    r.is_loss = v.at(4).as_bool();
    r.batch_size = v.at(5).as_int();
    return r;
}

mp::Value IRNode::pack() const {
    return mp::Value::array({mp::Value::str(name), packStrings(input_names), packStrings(output_names),
                             mp::Value::str(id), mp::Value::boolean(is_criterion), mp::Value::boolean(is_batch),
                             mp::Value::integer(batch_size)});
}
IRNode IRNode::unpack(const mp::Value& v) {
    IRNode n;
    n.name = v.at(0).as_str();
    n.input_names = unpackStrings(v.at(1));
    n.output_names = unpackStrings(v.at(2));
    n.id = v.at(3).as_str();
    n.is_criterion = v.at(4).as_bool();
    n.is_batch = v.at(5).as_bool();
    n.batch_size = v.at(6).as_int();
    return n;
}

// ---------------------------------------------------------------- IRGraph
const IRValue& IRGraph::value(const std::string& n) const {
    auto it = values.find(n);
    if (it == values.end()) throw std::runtime_error("IRGraph " + name + ": no value named " + n);
    return it->second;
}
IRValue& IRGraph::value(const std::string& n) {
    auto it = values.find(n);
    if (it == values.end()) throw std::runtime_error("IRGraph " + name + ": no value named " + n);
    return it->second;
}
bool IRGraph::isInput(const std::string& n) const {
    return std::find(input_names.begin(), input_names.end(), n) != input_names.end();
}
std::vector<std::string> IRGraph::paramInputNames() const {
    std::vector<std::string> r;
    for (const auto& n : input_names)
        if (value(n).is_param) r.push_back(n);
    return r;
}
std::vector<std::string> IRGraph::nonParamInputNames() const {
    std::vector<std::string> r;
    for (const auto& n : input_names)
        if (!value(n).is_param) r.push_back(n);
    return r;
}
int64_t IRGraph::paramSizeInByte() const {
    int64_t s = 0;
    for (const auto& n : input_names)
        if (value(n).is_param) s += value(n).type.sizeInByte();
    return s;
}
int64_t IRGraph::inputSizeInByte() const {
    int64_t s = 0;
    for (const auto& n : input_names)
        if (!value(n).is_param) s += value(n).type.sizeInByte();
    return s;
}
int64_t IRGraph::outputSizeInByte() const {
    int64_t s = 0;
    for (const auto& n : output_names) s += value(n).type.sizeInByte();
    return s;
}

int64_t IRGraph::commBufSize() const {
    int64_t in = 0, in_grad = 0;
    for (const auto& n : input_names) {
        const IRValue& v = value(n);
        if (v.is_param) continue;
        in += v.type.sizeInByte();
        if (v.type.holdsGradient()) in_grad += v.type.sizeInByte();
    }
    int64_t shared = 0;
    for (const auto& n : sharedInputs(*this)) {
        const IRValue& v = value(n);
        if (!v.is_param) shared += 2 * v.type.sizeInByte();
    }
    return in + outputSizeInByte() + in_grad + shared;
}

void IRGraph::check() const {
    std::unordered_set<std::string> defined(input_names.begin(), input_names.end());
    for (const auto& n : input_names)
        if (!values.count(n)) throw std::runtime_error("graph input without value: " + n);
    for (const auto& node : nodes) {
        for (const auto& in : node.input_names)
            if (!defined.count(in))
                throw std::runtime_error("node " + node.id + " reads " + in + " before it is defined");
        for (const auto& out : node.output_names) {
            if (!values.count(out)) throw std::runtime_error("node output without value: " + out);
            if (!defined.insert(out).second) throw std::runtime_error("value defined twice: " + out);
        }
    }
    for (const auto& o : output_names)
        if (!defined.count(o)) throw std::runtime_error("graph output never defined: " + o);
}

mp::Value IRGraph::pack() const {
    mp::Array ns;
    for (const auto& n : nodes) ns.push_back(n.pack());
    mp::MapItems vs;
    std::vector<std::string> keys;
    for (const auto& kv : values) keys.push_back(kv.first);
    std::sort(keys.begin(), keys.end());
    for (const auto& k : keys) vs.emplace_back(mp::Value::str(k), values.at(k).pack());
    return mp::Value::array({mp::Value::str(name), mp::Value::array(std::move(ns)), mp::Value::mapping(std::move(vs)),
                             packStrings(input_names), packStrings(output_names),
                             mp::Value::boolean(is_replicable), mp::Value::integer(batch_size)});
}

IRGraph IRGraph::unpack(const mp::Value& v) {
    IRGraph g;
    g.name = v.at(0).as_str();
    for (const auto& n : v.at(1).as_array()) g.nodes.push_back(IRNode::unpack(n));
    for (const auto& kv : v.at(2).as_map()) g.values[kv.first.as_str()] = IRValue::unpack(kv.second);
    g.input_names = unpackStrings(v.at(3));
    g.output_names = unpackStrings(v.at(4));
    g.is_replicable = v.at(5).as_bool();
    g.batch_size = v.at(6).as_int();
    return g;
}

static std::string typeToString(const IRType& t) {
    std::ostringstream ss;
    switch (t.base_type) {
        case IRBaseType::TENSOR: {
            ss << elemTypeName(t.tensor_elem_type) << "[";
            for (size_t i = 0; i < t.tensor_dim.size(); ++i) ss << (i ? "," : "") << t.tensor_dim[i];
            ss << "]";
            break;
        }
        case IRBaseType::SCALAR: ss << "scalar"; break;
        case IRBaseType::STRING: ss << "str"; break;
        case IRBaseType::LIST:
        case IRBaseType::TUPLE: {
            ss << (t.base_type == IRBaseType::LIST ? "list(" : "tuple(");
            for (size_t i = 0; i < t.compound_types.size(); ++i) ss << (i ? "," : "") << typeToString(t.compound_types[i]);
            ss << ")";
            break;
        }
        case IRBaseType::OPTIONAL: ss << "optional"; break;
        case IRBaseType::FUNCTION: ss << "fn:" << t.func_name; break;
        default: ss << "none";
    }
    return ss.str();
}

std::string IRGraph::toString() const {
    std::ostringstream ss;
    ss << "graph " << name << " (batch_size=" << batch_size << ")\n";
    for (const auto& n : input_names) {
        const IRValue& v = value(n);
        ss << "  in  " << n << " : " << typeToString(v.type) << (v.is_param ? " param" : "")
           << (v.is_batch ? " batch" : "") << "\n";
    }
    for (const auto& node : nodes) {
        ss << "  " << node.id << " = " << node.name << "(";
        for (size_t i = 0; i < node.input_names.size(); ++i) ss << (i ? ", " : "") << node.input_names[i];
        ss << ") -> ";
        for (size_t i = 0; i < node.output_names.size(); ++i)
            ss << (i ? ", " : "") << node.output_names[i] << ":" << typeToString(value(node.output_names[i]).type);
        if (node.is_criterion) ss << " [criterion]";
        else if (node.is_batch) ss << " [batch]";
        ss << "\n";
    }
    for (const auto& n : output_names) ss << "  out " << n << "\n";
    return ss.str();
}

std::string IRGraph::toDot() const {
    std::ostringstream ss;
    ss << "digraph \"" << name << "\" {\n";
    for (const auto& kv : values)
        ss << "  \"v_" << kv.first << "\" [shape=ellipse,label=\"" << kv.first << "\\n" << typeToString(kv.second.type)
           << "\"" << (kv.second.is_param ? ",style=filled,fillcolor=lightgrey" : "") << "];\n";
    for (const auto& n : nodes) {
        ss << "  \"n_" << n.id << "\" [shape=box,label=\"" << n.name << "\"];\n";
        for (const auto& in : n.input_names) ss << "  \"v_" << in << "\" -> \"n_" << n.id << "\";\n";
        for (const auto& out : n.output_names) ss << "  \"n_" << n.id << "\" -> \"v_" << out << "\";\n";
    }
    ss << "}\n";
    return ss.str();
}

std::unordered_map<std::string, std::vector<size_t>> consumers(const IRGraph& g) {
    std::unordered_map<std::string, std::vector<size_t>> r;
    for (size_t i = 0; i < g.nodes.size(); ++i)
        for (const auto& in : g.nodes[i].input_names) {
            auto& v = r[in];
            if (v.empty() || v.back() != i) v.push_back(i);
        }
    return r;
}
std::unordered_map<std::string, size_t> producers(const IRGraph& g) {
    std::unordered_map<std::string, size_t> r;
    for (size_t i = 0; i < g.nodes.size(); ++i)
        for (const auto& out : g.nodes[i].output_names) r[out] = i;
    return r;
}

std::vector<std::string> findUnusedValues(const IRGraph& g) {
    auto cons = consumers(g);
    std::unordered_set<std::string> outs(g.output_names.begin(), g.output_names.end());
    std::vector<std::string> unused;
    for (const auto& kv : g.values)
        if (!cons.count(kv.first) && !outs.count(kv.first)) unused.push_back(kv.first);
    std::sort(unused.begin(), unused.end());
    return unused;
}

IRGraph removeUnusedNodes(const IRGraph& g) {
    std::unordered_set<std::string> live(g.output_names.begin(), g.output_names.end());
    std::vector<bool> keep(g.nodes.size(), false);
    for (size_t k = g.nodes.size(); k-- > 0;) {
        const IRNode& n = g.nodes[k];
        bool used = false;
        for (const auto& o : n.output_names)
            if (live.count(o)) used = true;
        if (!used) continue;
        keep[k] = true;
        for (const auto& in : n.input_names) live.insert(in);
    }
    IRGraph r;
    r.name = g.name;
    r.is_replicable = g.is_replicable;
    r.batch_size = g.batch_size;
    r.output_names = g.output_names;
    for (const auto& in : g.input_names)
        if (live.count(in)) {
            r.input_names.push_back(in);
            r.values[in] = g.value(in);
        }
    for (size_t k = 0; k < g.nodes.size(); ++k)
        if (keep[k]) {
            r.nodes.push_back(g.nodes[k]);
            for (const auto& o : g.nodes[k].output_names) r.values[o] = g.value(o);
        }
    return r;
}

IRGraph scaleGraph(const IRGraph& g, int64_t new_bs) {
    IRGraph r = g;
    if (g.batch_size <= 0 || new_bs == g.batch_size) return r;
    for (auto& kv : r.values) {
        if (kv.second.is_batch) {
            kv.second.type.scaleBatch(new_bs, g.batch_size);
            kv.second.batch_size = new_bs;
        }
    }
    for (auto& n : r.nodes)
        if (n.is_batch) n.batch_size = new_bs;
    r.batch_size = new_bs;
    return r;
}

std::vector<std::string> sharedInputs(const IRGraph& g) {
    std::unordered_map<std::string, int> uses;
    for (const auto& n : g.nodes) {
        std::unordered_set<std::string> seen;
        for (const auto& in : n.input_names)
            if (seen.insert(in).second) uses[in]++;
    }
    std::vector<std::string> r;
    for (const auto& in : g.input_names)
        if (uses[in] > 1) r.push_back(in);
    return r;
}

// ---------------------------------------------------------------- value classification
namespace {
enum class VClass { CONST_, BATCH, PARAM, LOSS };

bool isTensorLike(const IRType& t) {
    if (t.base_type == IRBaseType::TENSOR) return true;
    if (t.base_type == IRBaseType::LIST || t.base_type == IRBaseType::TUPLE)
        for (const auto& c : t.compound_types)
            if (isTensorLike(c)) return true;
    return false;
}
bool isScalarTensor(const IRType& t) { return t.base_type == IRBaseType::TENSOR && t.tensor_dim.empty(); }
}  // namespace

void guessValueTypes(IRGraph& g) {
    std::unordered_map<std::string, VClass> cls;
    for (const auto& in : g.input_names) {
        const IRValue& v = g.value(in);
        if (v.is_param) cls[in] = VClass::PARAM;
        else if (isTensorLike(v.type)) cls[in] = VClass::BATCH;
        else cls[in] = VClass::CONST_;
    }
    for (auto& node : g.nodes) {
        int n_batch = 0, n_loss = 0, n_param = 0;
        std::unordered_set<std::string> seen;
        for (const auto& in : node.input_names) {
            if (!seen.insert(in).second) continue;
            auto it = cls.find(in);
            const VClass c = it == cls.end() ? VClass::CONST_ : it->second;
            if (c == VClass::BATCH) ++n_batch;
            else if (c == VClass::LOSS) ++n_loss;
            else if (c == VClass::PARAM) ++n_param;
        }
        bool tensor_out = false;
        for (const auto& o : node.output_names)
            if (isTensorLike(g.value(o).type)) tensor_out = true;
        const bool single_scalar =
            node.output_names.size() == 1 && isScalarTensor(g.value(node.output_names[0]).type);
        VClass c;
        if (single_scalar && ((n_loss > 0 && n_batch == 0) || n_batch == 2)) c = VClass::LOSS;
        else if (n_batch > 0 && tensor_out) c = VClass::BATCH;
        else if (n_loss > 0 && single_scalar) c = VClass::LOSS;
        else if (n_param == 1) c = VClass::PARAM;
        else c = VClass::CONST_;
        node.is_criterion = c == VClass::LOSS;
        node.is_batch = c == VClass::BATCH;
        node.batch_size = (c == VClass::BATCH || c == VClass::LOSS) ? g.batch_size : 0;
        for (const auto& o : node.output_names) cls[o] = c;
    }
    for (auto& kv : g.values) {
        auto it = cls.find(kv.first);
        const VClass c = it == cls.end() ? VClass::CONST_ : it->second;
        // A tensor computed from batch values whose shape holds no batch dimension (mean over the batch, a
        // running statistic) stays in the batch flow as far as node ownership goes (its node is placed in
        // exactly one stage), but the value itself is moved whole, not split into rows.
        const bool whole = c == VClass::BATCH && kv.second.batch_hint < 0;
        kv.second.is_batch = c == VClass::BATCH && !whole;
        kv.second.is_loss = c == VClass::LOSS;
        kv.second.batch_size = ((c == VClass::BATCH && !whole) || c == VClass::LOSS) ? g.batch_size : 0;
    }
}

// ---------------------------------------------------------------- IValueLocation
mp::Value IValueLocation::pack() const {
    mp::Array p;
    for (const auto& s : path)
        p.push_back(mp::Value::array({mp::Value::integer(s.type), mp::Value::integer(s.index)}));
    return mp::Value::array({mp::Value::str(value_name), mp::Value::array(std::move(p))});
}
IValueLocation IValueLocation::unpack(const mp::Value& v) {
    IValueLocation l;
    l.value_name = v.at(0).as_str();
    for (const auto& s : v.at(1).as_array()) {
        StepInIValue st;
        st.type = static_cast<int>(s.at(0).as_int());
        st.index = s.at(1).as_int();
        l.path.push_back(st);
    }
    return l;
}
std::string IValueLocation::toString() const {
    std::ostringstream ss;
    ss << value_name;
    for (const auto& s : path) ss << (s.type == 0 ? "[L" : "[T") << s.index << "]";
    return ss.str();
}
bool IValueLocation::operator==(const IValueLocation& o) const {
    if (value_name != o.value_name || path.size() != o.path.size()) return false;
    for (size_t i = 0; i < path.size(); ++i)
        if (path[i].type != o.path[i].type || path[i].index != o.path[i].index) return false;
    return true;
}

}  // namespace rannc
