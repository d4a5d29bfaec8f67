// Package loader (declarations and contract: include/vxb200_package.h): graph.json +
// SafeTensors -> validated node list -> repacked weights on the device -> forward passes whose
// intermediate tensors stay in HBM.  Host code only; every kernel is reached through the C ABI
// of include/vxb200_w8a8.h.
//
// Reference counterparts: the SafeTensors reader native/src/runtime/safetensors.c (8-byte
// little-endian header length, JSON header {name: {dtype, shape, data_offsets}}, "__metadata__"
// ignored as authority), the affine metadata contract docs/w8a8-safetensors.md:13-121, the dense
// layout rule docs/model-format.md:280-287, PackedLinear nodes as the exporter writes them
// (tools/exporter/packed_linear.py:160-205) and the storage contract
// docs/packed-linear-design.md:24-41.
#include "../../include/vxb200_package.h"
#include "common.cuh"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

using namespace vxb;

namespace {

// ---- a small JSON reader (objects keep their member order) -----------------------------------
struct Json {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    bool boolean = false;
    double number = 0.0;
    bool integral = false;   // the number was written without fraction or exponent
    std::string text;
    std::vector<Json> items;
    std::vector<std::pair<std::string, Json>> members;
    const Json* get(const char* key) const {
        if (kind != Object) return nullptr;
        for (auto& m : members) if (m.first == key) return &m.second;
        return nullptr;
    }
    bool is_string() const { return kind == String; }
    bool is_int() const { return kind == Number && integral; }
};

struct JsonParser {
    const char* p; const char* end; std::string error;
    void skip() { while (p < end && (*p == ' ' || *p == '\t' || *p == '\n' || *p == '\r')) p++; }
    bool fail(const char* what) { if (error.empty()) error = what; return false; }
    bool parse_string(std::string& out) {
        if (p >= end || *p != '"') return fail("expected a string");
        p++;
        while (p < end && *p != '"') {
            if ((unsigned char)*p < 0x20) return fail("control character in a string");
            if (*p == '\\') {
                if (++p >= end) return fail("unterminated escape");
                switch (*p) {
                    case '"': out += '"'; break; case '\\': out += '\\'; break; case '/': out += '/'; break;
                    case 'b': out += '\b'; break; case 'f': out += '\f'; break; case 'n': out += '\n'; break;
                    case 'r': out += '\r'; break; case 't': out += '\t'; break;
                    case 'u': {
                        if (end - p < 5) return fail("short \\u escape");
                        unsigned v = 0;
                        for (int i = 1; i <= 4; i++) {
                            const char c = p[i];
                            v = v * 16 + (c >= '0' && c <= '9' ? c - '0' : c >= 'a' && c <= 'f' ? c - 'a' + 10 : c >= 'A' && c <= 'F' ? c - 'A' + 10 : 256);
                            if (v > 0xffff) return fail("bad \\u escape");
                        }
                        p += 4;
                        if (v < 0x80) out += (char)v;
                        else if (v < 0x800) { out += (char)(0xc0 | (v >> 6)); out += (char)(0x80 | (v & 0x3f)); }
                        else { out += (char)(0xe0 | (v >> 12)); out += (char)(0x80 | ((v >> 6) & 0x3f)); out += (char)(0x80 | (v & 0x3f)); }
                        break;
                    }
                    default: return fail("unknown escape");
                }
                p++;
            } else out += *p++;
        }
        if (p >= end) return fail("unterminated string");
        p++;
        return true;
    }
    bool parse(Json& out, int depth = 0) {
        if (depth > 64) return fail("nesting too deep");
        skip();
        if (p >= end) return fail("unexpected end");
        if (*p == '{') {
            out.kind = Json::Object; p++; skip();
            if (p < end && *p == '}') { p++; return true; }
            for (;;) {
                skip();
                std::string key;
                if (!parse_string(key)) return false;
                for (auto& m : out.members) if (m.first == key) return fail("duplicate object key");
                skip();
                if (p >= end || *p != ':') return fail("expected ':'");
                p++;
                out.members.emplace_back(key, Json());
                if (!parse(out.members.back().second, depth + 1)) return false;
                skip();
                if (p < end && *p == ',') { p++; continue; }
                if (p < end && *p == '}') { p++; return true; }
                return fail("expected ',' or '}'");
            }
        }
        if (*p == '[') {
            out.kind = Json::Array; p++; skip();
            if (p < end && *p == ']') { p++; return true; }
            for (;;) {
                out.items.emplace_back();
                if (!parse(out.items.back(), depth + 1)) return false;
                skip();
                if (p < end && *p == ',') { p++; continue; }
                if (p < end && *p == ']') { p++; return true; }
                return fail("expected ',' or ']'");
            }
        }
        if (*p == '"') { out.kind = Json::String; return parse_string(out.text); }
        if (end - p >= 4 && !strncmp(p, "true", 4)) { out.kind = Json::Bool; out.boolean = true; p += 4; return true; }
        if (end - p >= 5 && !strncmp(p, "false", 5)) { out.kind = Json::Bool; p += 5; return true; }
        if (end - p >= 4 && !strncmp(p, "null", 4)) { out.kind = Json::Null; p += 4; return true; }
        const char* start = p;
        if (p < end && *p == '-') p++;
        if (p >= end || *p < '0' || *p > '9') return fail("unexpected character");
        while (p < end && *p >= '0' && *p <= '9') p++;
        bool integral = true;
        if (p < end && *p == '.') { integral = false; p++; while (p < end && *p >= '0' && *p <= '9') p++; }
        if (p < end && (*p == 'e' || *p == 'E')) {
            integral = false; p++;
            if (p < end && (*p == '+' || *p == '-')) p++;
            while (p < end && *p >= '0' && *p <= '9') p++;
        }
        out.kind = Json::Number; out.integral = integral;
        out.number = strtod(std::string(start, p).c_str(), nullptr);
        return true;
    }
};

bool parse_json(const char* data, size_t bytes, Json& out, std::string& error) {
    JsonParser parser{data, data + bytes, {}};
    if (!parser.parse(out)) { error = parser.error; return false; }
    parser.skip();
    if (parser.p != parser.end) { error = "trailing characters after the JSON document"; return false; }
    return true;
}

bool read_file(const char* path, std::vector<unsigned char>& out) {
    FILE* f = fopen(path, "rb");
    if (!f) return false;
    bool ok = fseek(f, 0, SEEK_END) == 0;
    const long size = ok ? ftell(f) : -1;
    ok = ok && size >= 0 && fseek(f, 0, SEEK_SET) == 0;
    if (ok) { out.resize((size_t)size); ok = size == 0 || fread(out.data(), 1, (size_t)size, f) == (size_t)size; }
    fclose(f);
    return ok;
}

// ---- tensors -------------------------------------------------------------------------------------
enum DType : uint32_t { kF32 = VXB_DTYPE_F32, kU8 = VXB_DTYPE_U8, kI8 = VXB_DTYPE_I8, kI32 = VXB_DTYPE_I32 };
size_t dtype_bytes(uint32_t dt) { return dt == kF32 || dt == kI32 ? 4 : 1; }

struct StoredTensor {           // one SafeTensors entry, pointing into its file's bytes
    uint32_t dtype = 0;
    std::vector<int64_t> shape;
    const unsigned char* data = nullptr;
    size_t bytes = 0;
    size_t elements() const { size_t n = 1; for (int64_t d : shape) n *= (size_t)d; return n; }
};

struct GraphTensor {            // an activation: a graph input or a node output
    std::string name;
    uint32_t dtype = 0;
    std::vector<int64_t> shape;
    size_t elements() const { size_t n = 1; for (int64_t d : shape) n *= (size_t)d; return n; }
    size_t bytes() const { return elements() * dtype_bytes(dtype); }
    uint32_t rows() const { size_t n = 1; for (size_t i = 0; i + 1 < shape.size(); i++) n *= (size_t)shape[i]; return (uint32_t)n; }
    uint32_t width() const { return shape.empty() ? 1u : (uint32_t)shape.back(); }
};

struct Affine { float scale = 1.0f; int32_t zero = 0; };   // per-tensor descriptor, resolved

enum Op { kQuantize, kDequantize, kRequantize, kQLinear, kPackedLinear };

struct Node {
    std::string id, op_name;
    Op op;
    int input = -1, output = -1;            // indices into VxbPackage::tensors
    Affine in_q, out_q;                     // resolved per-tensor metadata of byte tensors
    // QLinear
    const StoredTensor* weight = nullptr; const StoredTensor* weight_scale = nullptr; const StoredTensor* bias = nullptr;
    // PackedLinear
    const StoredTensor* words = nullptr; const StoredTensor* group_scales = nullptr; const StoredTensor* bias_f32 = nullptr;
    uint32_t weight_bits = 0, group_size = 0, d_in = 0, d_out = 0;
};

}  // namespace

struct VxbPackage {
    std::vector<std::vector<unsigned char>> files;          // SafeTensors files, kept whole
    std::map<std::string, StoredTensor> stored;
    std::vector<GraphTensor> tensors;                       // activations in creation order
    std::map<std::string, int> tensor_index;
    std::vector<int> inputs, outputs;
    std::vector<Node> nodes;
};

struct VxbProgram {
    VxbContext* ctx = nullptr;
    std::vector<GraphTensor> tensors;
    std::vector<int> inputs, outputs;
    std::vector<Node> nodes;                                // weight pointers are not used after compile
    std::vector<VxbWeight*> weights;                        // per node (null for boundary ops)
    std::vector<void*> buffers;                             // device buffer per tensor
    uint64_t device_bytes = 0;
    std::string evidence;
};

namespace {

bool parse_dtype_graph(const std::string& s, uint32_t* dt) {
    if (s == "float32") *dt = kF32; else if (s == "int8") *dt = kI8; else if (s == "uint8") *dt = kU8; else if (s == "int32") *dt = kI32;
    else return false;
    return true;
}

// One SafeTensors file: u64 little-endian header length, JSON header, then the data section.
int load_safetensors(VxbPackage& pkg, const char* path) {
    pkg.files.emplace_back();
    std::vector<unsigned char>& file = pkg.files.back();
    if (!read_file(path, file)) return set_error(0, "cannot read %s", path);
    if (file.size() < 8) return set_error(0, "%s: shorter than a SafeTensors header", path);
    uint64_t header_bytes = 0;
    for (int i = 7; i >= 0; i--) header_bytes = (header_bytes << 8) | file[i];
    if (header_bytes == 0 || header_bytes > 100000000ull || header_bytes > file.size() - 8)
        return set_error(0, "%s: header length %llu outside the file", path, (unsigned long long)header_bytes);
    Json header; std::string error;
    if (!parse_json((const char*)file.data() + 8, (size_t)header_bytes, header, error) || header.kind != Json::Object)
        return set_error(0, "%s: header is not a JSON object (%s)", path, error.c_str());
    const unsigned char* data = file.data() + 8 + header_bytes;
    const size_t data_bytes = file.size() - 8 - (size_t)header_bytes;
    std::vector<std::pair<size_t, size_t>> ranges;
    for (auto& m : header.members) {
        if (m.first == "__metadata__") {
            if (m.second.kind != Json::Object) return set_error(0, "%s: __metadata__ is not an object", path);
            for (auto& kv : m.second.members) {
                if (!kv.second.is_string()) return set_error(0, "%s: __metadata__ values must be strings", path);
                // retired quantization metadata is invalid (docs/w8a8-safetensors.md:99-101)
                if (kv.first == "weights_quantization" || kv.first == "weights_quantization_storage")
                    return set_error(0, "%s: retired metadata key %s", path, kv.first.c_str());
            }
            continue;
        }
        const Json* dt = m.second.get("dtype"); const Json* shape = m.second.get("shape"); const Json* off = m.second.get("data_offsets");
        if (m.second.kind != Json::Object || m.second.members.size() != 3 || !dt || !dt->is_string() || !shape ||
            shape->kind != Json::Array || !off || off->kind != Json::Array || off->items.size() != 2 ||
            !off->items[0].is_int() || !off->items[1].is_int())
            return set_error(0, "%s: malformed entry for tensor %s", path, m.first.c_str());
        StoredTensor t;
        if (dt->text == "F32") t.dtype = kF32; else if (dt->text == "I8") t.dtype = kI8; else if (dt->text == "U8") t.dtype = kU8;
        else if (dt->text == "I32") t.dtype = kI32;
        else t.dtype = 0;   // another dtype: legal in the file, unusable by the operators served here
        size_t elements = 1;
        for (auto& d : shape->items) {
            if (!d.is_int() || d.number < 0 || d.number > 9007199254740991.0) return set_error(0, "%s: bad shape of %s", path, m.first.c_str());
            t.shape.push_back((int64_t)d.number);
            if (d.number != 0 && elements > (size_t)-1 / (size_t)d.number) return set_error(0, "%s: shape of %s overflows", path, m.first.c_str());
            elements *= (size_t)d.number;
        }
        const double b = off->items[0].number, e = off->items[1].number;
        if (b < 0 || e < b || e > (double)data_bytes) return set_error(0, "%s: data_offsets of %s outside the file", path, m.first.c_str());
        t.data = data + (size_t)b; t.bytes = (size_t)(e - b);
        if (t.dtype && t.bytes != elements * dtype_bytes(t.dtype))
            return set_error(0, "%s: tensor %s has %zu bytes for %zu elements", path, m.first.c_str(), t.bytes, elements);
        ranges.emplace_back((size_t)b, (size_t)e);
        if (pkg.stored.count(m.first)) return set_error(0, "tensor name %s is not unique in the weight set", m.first.c_str());
        pkg.stored[m.first] = t;
    }
    // the data section is covered exactly once, without holes or overlap
    std::sort(ranges.begin(), ranges.end());
    size_t at = 0;
    for (auto& r : ranges) { if (r.first != at) return set_error(0, "%s: tensor data has a hole or an overlap at byte %zu", path, at); at = r.second; }
    if (at != data_bytes) return set_error(0, "%s: %zu trailing bytes after the last tensor", path, data_bytes - at);
    return 1;
}

const StoredTensor* stored(const VxbPackage& pkg, const Json* name, uint32_t dtype, size_t rank) {
    if (!name || !name->is_string()) return nullptr;
    auto it = pkg.stored.find(name->text);
    if (it == pkg.stored.end() || it->second.dtype != dtype || it->second.shape.size() != rank) return nullptr;
    return &it->second;
}

// Per-tensor affine descriptor of the byte tensor `target` from the central table: F32 scale [1],
// zero point [1] of the target's own dtype, scale finite and positive.
int resolve_per_tensor(const VxbPackage& pkg, const Json* table, const GraphTensor& target, Affine* out,
                       std::string* scale_name, std::string* zero_name) {
    const Json* d = table ? table->get(target.name.c_str()) : nullptr;
    if (!d || d->kind != Json::Object) return set_error(0, "byte tensor %s has no affine descriptor", target.name.c_str());
    const Json* scheme = d->get("scheme");
    if (!scheme || !scheme->is_string() || scheme->text != "per_tensor" || d->members.size() != 3)
        return set_error(0, "descriptor of %s is not {scheme: per_tensor, scale_tensor, zero_point_tensor}", target.name.c_str());
    const Json* sn = d->get("scale_tensor"); const Json* zn = d->get("zero_point_tensor");
    const StoredTensor* s = stored(pkg, sn, kF32, 1); const StoredTensor* z = stored(pkg, zn, target.dtype, 1);
    if (!s || !z || s->shape[0] != 1 || z->shape[0] != 1 || sn->text == zn->text)
        return set_error(0, "scale / zero point of %s do not resolve to F32 [1] and a [1] tensor of its own dtype", target.name.c_str());
    memcpy(&out->scale, s->data, 4);
    out->zero = target.dtype == kU8 ? (int32_t)z->data[0] : (int32_t)(int8_t)z->data[0];
    if (!std::isfinite(out->scale) || !(out->scale > 0.0f)) return set_error(0, "scale of %s is not finite and positive", target.name.c_str());
    if (scale_name) *scale_name = sn->text;
    if (zero_name) *zero_name = zn->text;
    return 1;
}

int parse_shape(const Json* shape, std::vector<int64_t>* out, const char* what) {
    if (!shape || shape->kind != Json::Array || shape->items.empty() || shape->items.size() > 8) return set_error(0, "%s: bad shape", what);
    for (auto& d : shape->items) {
        if (d.is_string()) return set_error(0, "%s: symbolic dimension %s is not served (fixed shapes only)", what, d.text.c_str());
        if (!d.is_int() || d.number < 1 || d.number > 2147483647.0) return set_error(0, "%s: bad dimension", what);
        out->push_back((int64_t)d.number);
    }
    return 1;
}

int add_tensor(VxbPackage& pkg, const std::string& name, uint32_t dtype, const std::vector<int64_t>& shape) {
    if (pkg.tensor_index.count(name) || pkg.stored.count(name)) return set_error(0, "tensor name %s is defined twice", name.c_str());
    GraphTensor t; t.name = name; t.dtype = dtype; t.shape = shape;
    pkg.tensor_index[name] = (int)pkg.tensors.size();
    pkg.tensors.push_back(t);
    return 1;
}

int build_graph(VxbPackage& pkg, const Json& g) {
    const Json* format = g.get("format");
    if (!format || !format->is_string() || format->text != "volvox-graph/v1") return set_error(0, "graph format is not volvox-graph/v1");
    for (const char* retired : {"weights_quantization", "weights_quantization_storage"})
        if (g.get(retired)) return set_error(0, "retired graph field %s", retired);
    const Json* inputs = g.get("inputs"); const Json* nodes = g.get("nodes"); const Json* outputs = g.get("outputs");
    if (!inputs || inputs->kind != Json::Object || !nodes || nodes->kind != Json::Array || !outputs || outputs->kind != Json::Array)
        return set_error(0, "graph needs inputs, nodes and outputs");
    const Json* quant = g.get("quantization");
    const Json* table = nullptr;
    if (quant) {
        const Json* qf = quant->get("format");
        table = quant->get("tensors");
        if (quant->kind != Json::Object || quant->members.size() != 2 || !qf || !qf->is_string() ||
            qf->text != "volvox-affine-safetensors/v1" || !table || table->kind != Json::Object || table->members.empty())
            return set_error(0, "quantization must be {format: volvox-affine-safetensors/v1, tensors: {...}}");
    }
    for (auto& in : inputs->members) {
        if (in.second.get("quantization")) return set_error(0, "input %s carries an inline quantization value", in.first.c_str());
        const Json* dt = in.second.get("dtype");
        uint32_t dtype; std::vector<int64_t> shape;
        if (!dt || !dt->is_string() || !parse_dtype_graph(dt->text, &dtype) || dtype == kI32)
            return set_error(0, "input %s: dtype must be float32, int8 or uint8", in.first.c_str());
        if (parse_shape(in.second.get("shape"), &shape, in.first.c_str()) != 1) return 0;
        if (add_tensor(pkg, in.first, dtype, shape) != 1) return 0;
        pkg.inputs.push_back(pkg.tensor_index[in.first]);
    }
    if (pkg.inputs.empty()) return set_error(0, "graph has no inputs");
    for (auto& jn : nodes->items) {
        Node node;
        const Json* id = jn.get("id"); const Json* op = jn.get("opType"); const Json* in = jn.get("inputs");
        const Json* outs = jn.get("outputs"); const Json* params = jn.get("params");
        if (!id || !id->is_string() || !op || !op->is_string() || !in || in->kind != Json::Object || !outs || outs->kind != Json::Object)
            return set_error(0, "malformed node");
        if (jn.get("outputs_quantization")) return set_error(0, "node %s carries outputs_quantization", id->text.c_str());
        node.id = id->text; node.op_name = op->text;
        const char* nid = node.id.c_str();
        if (op->text == "QuantizeLinear") node.op = kQuantize; else if (op->text == "DequantizeLinear") node.op = kDequantize;
        else if (op->text == "RequantizeLinear") node.op = kRequantize; else if (op->text == "QLinear") node.op = kQLinear;
        else if (op->text == "PackedLinear") node.op = kPackedLinear;
        else return set_error(0, "node %s: operator %s is not served by this route", nid, op->text.c_str());
        const Json* x = in->get("input");
        if (!x || !x->is_string() || !pkg.tensor_index.count(x->text)) return set_error(0, "node %s: input does not name an activation defined before it", nid);
        node.input = pkg.tensor_index[x->text];
        const GraphTensor xin = pkg.tensors[node.input];
        const Json* out = outs->get("out");
        const Json* oname = out ? out->get("tensor") : nullptr; const Json* odt = out ? out->get("dtype") : nullptr;
        uint32_t out_dtype; std::vector<int64_t> out_shape;
        if (outs->members.size() != 1 || !oname || !oname->is_string() || !odt || !odt->is_string() || !parse_dtype_graph(odt->text, &out_dtype))
            return set_error(0, "node %s: outputs must be {out: {tensor, shape, dtype}}", nid);
        if (parse_shape(out->get("shape"), &out_shape, nid) != 1) return 0;
        if (add_tensor(pkg, oname->text, out_dtype, out_shape) != 1) return 0;
        node.output = pkg.tensor_index[oname->text];
        const GraphTensor& yout = pkg.tensors[node.output];
        const bool in_byte = xin.dtype == kI8 || xin.dtype == kU8, out_byte = out_dtype == kI8 || out_dtype == kU8;
        const size_t expected_inputs = node.op == kQuantize || node.op == kDequantize ? 3 : node.op == kRequantize ? 1 : 0;
        switch (node.op) {
            case kQuantize: case kDequantize: {
                // Q/DQ operands must be the very tensors the central descriptor names
                const GraphTensor& byte_side = node.op == kQuantize ? yout : xin;
                const bool typed = node.op == kQuantize ? (xin.dtype == kF32 && out_byte) : (in_byte && out_dtype == kF32);
                if (!typed || in->members.size() != expected_inputs || xin.shape != yout.shape)
                    return set_error(0, "node %s: %s takes {input, scale, zero_point} and keeps the shape", nid, op->text.c_str());
                std::string sname, zname;
                Affine a;
                if (resolve_per_tensor(pkg, table, byte_side, &a, &sname, &zname) != 1) return 0;
                const Json* s = in->get("scale"); const Json* z = in->get("zero_point");
                if (!s || !s->is_string() || !z || !z->is_string() || s->text != sname || z->text != zname)
                    return set_error(0, "node %s: scale / zero_point operands differ from the central descriptor of %s", nid, byte_side.name.c_str());
                (node.op == kQuantize ? node.out_q : node.in_q) = a;
                break;
            }
            case kRequantize:
                if (!in_byte || !out_byte || in->members.size() != expected_inputs || xin.shape != yout.shape)
                    return set_error(0, "node %s: RequantizeLinear maps a byte tensor to a byte tensor of the same shape", nid);
                if (resolve_per_tensor(pkg, table, xin, &node.in_q, nullptr, nullptr) != 1 ||
                    resolve_per_tensor(pkg, table, yout, &node.out_q, nullptr, nullptr) != 1) return 0;
                break;
            case kQLinear: {
                if (params && !(params->kind == Json::Object && params->members.empty()))
                    return set_error(0, "node %s: QLinear params must be empty (the layout is fixed: dout_din)", nid);
                if (!in_byte || !out_byte || in->members.size() != 3) return set_error(0, "node %s: QLinear takes byte activations and {input, weight, bias}", nid);
                const Json* wn = in->get("weight");
                node.weight = stored(pkg, wn, kI8, 2);
                node.bias = stored(pkg, in->get("bias"), kI32, 1);
                if (!node.weight || !node.bias) return set_error(0, "node %s: weight must be I8 [d_out,d_in] and bias I32 [d_out]", nid);
                node.d_out = (uint32_t)node.weight->shape[0]; node.d_in = (uint32_t)node.weight->shape[1];
                if ((int64_t)node.d_in != xin.shape.back() || (int64_t)node.d_out != yout.shape.back() || node.bias->shape[0] != node.d_out ||
                    xin.rows() != yout.rows())
                    return set_error(0, "node %s: shapes of input, weight, bias and output disagree", nid);
                // weight descriptor: per_axis on axis 0 (a negative spelling is normalised), F32 scales [d_out],
                // explicit I8 zero points [d_out], all zero
                const Json* d = table ? table->get(wn->text.c_str()) : nullptr;
                const Json* scheme = d ? d->get("scheme") : nullptr; const Json* axis = d ? d->get("axis") : nullptr;
                if (!d || d->members.size() != 4 || !scheme || !scheme->is_string() || scheme->text != "per_axis" || !axis || !axis->is_int() ||
                    !(axis->number == 0 || axis->number == -2))
                    return set_error(0, "node %s: the weight needs a per_axis descriptor on axis 0", nid);
                node.weight_scale = stored(pkg, d->get("scale_tensor"), kF32, 1);
                const StoredTensor* wz = stored(pkg, d->get("zero_point_tensor"), kI8, 1);
                if (!node.weight_scale || !wz || node.weight_scale->shape[0] != node.d_out || wz->shape[0] != node.d_out ||
                    d->get("scale_tensor")->text == d->get("zero_point_tensor")->text)
                    return set_error(0, "node %s: weight scale / zero point must be F32 [d_out] and I8 [d_out]", nid);
                for (uint32_t i = 0; i < node.d_out; i++) {
                    float s; memcpy(&s, node.weight_scale->data + 4 * (size_t)i, 4);
                    if (!std::isfinite(s) || !(s > 0.0f)) return set_error(0, "node %s: weight scale %u is not finite and positive", nid, i);
                    if (wz->data[i] != 0) return set_error(0, "node %s: non-zero weight zero point at channel %u (stays with the reference's routes)", nid, i);
                }
                if (resolve_per_tensor(pkg, table, xin, &node.in_q, nullptr, nullptr) != 1 ||
                    resolve_per_tensor(pkg, table, yout, &node.out_q, nullptr, nullptr) != 1) return 0;
                break;
            }
            case kPackedLinear: {
                const Json* gs = params ? params->get("group_size") : nullptr; const Json* wb = params ? params->get("weight_bits") : nullptr;
                if (!params || params->members.size() != 2 || !gs || !gs->is_int() || !wb || !wb->is_int())
                    return set_error(0, "node %s: PackedLinear params must be {group_size, weight_bits}", nid);
                node.group_size = (uint32_t)gs->number; node.weight_bits = (uint32_t)wb->number;
                if (node.group_size != 32 && node.group_size != 64 && node.group_size != 128 && node.group_size != 256)
                    return set_error(0, "node %s: group size %u is not 32/64/128/256", nid, node.group_size);
                if (node.weight_bits != 8 && node.weight_bits != 4)
                    return set_error(0, "node %s: weight bits %u stay with the reference's routes (8 and 4 are served)", nid, node.weight_bits);
                if (xin.dtype != kF32 || out_dtype != kF32) return set_error(0, "node %s: PackedLinear activations are float32", nid);
                node.words = stored(pkg, in->get("weight"), kI32, 2);
                node.group_scales = stored(pkg, in->get("scale"), kF32, 2);
                const Json* bn = in->get("bias");
                if (bn) { node.bias_f32 = stored(pkg, bn, kF32, 1); if (!node.bias_f32) return set_error(0, "node %s: bias must be F32 [N]", nid); }
                if (!node.words || !node.group_scales || in->members.size() != (bn ? 4u : 3u))
                    return set_error(0, "node %s: PackedLinear takes {input, weight (I32 words), scale (F32), bias?}", nid);
                node.d_in = (uint32_t)xin.shape.back(); node.d_out = (uint32_t)node.words->shape[0];
                const uint32_t row_words = (node.d_in * node.weight_bits + 31) / 32, groups = (node.d_in + node.group_size - 1) / node.group_size;
                if (node.words->shape[1] != row_words || node.group_scales->shape[0] != node.d_out || node.group_scales->shape[1] != groups ||
                    (int64_t)node.d_out != yout.shape.back() || (node.bias_f32 && node.bias_f32->shape[0] != node.d_out) || xin.rows() != yout.rows())
                    return set_error(0, "node %s: words must be [N, ceil(K*bits/32)], scales [N, ceil(K/G)] for the input's K", nid);
                break;
            }
        }
        pkg.nodes.push_back(node);
    }
    if (pkg.nodes.empty()) return set_error(0, "graph has no nodes");
    for (auto& o : outputs->items) {
        if (!o.is_string() || !pkg.tensor_index.count(o.text)) return set_error(0, "graph output does not name a tensor");
        pkg.outputs.push_back(pkg.tensor_index[o.text]);
    }
    if (pkg.outputs.empty()) return set_error(0, "graph has no outputs");
    // a quantization parameter must not itself have an affine descriptor
    if (table)
        for (auto& d : table->members) {
            for (const char* key : {"scale_tensor", "zero_point_tensor"}) {
                const Json* ref = d.second.get(key);
                if (ref && ref->is_string() && table->get(ref->text.c_str()))
                    return set_error(0, "quantization parameter %s has an affine descriptor of its own", ref->text.c_str());
            }
            if (!pkg.tensor_index.count(d.first) && !pkg.stored.count(d.first))
                return set_error(0, "descriptor target %s is not a tensor of this graph", d.first.c_str());
        }
    return 1;
}

const std::vector<int>& io_list(const VxbPackage* p, int is_output) { return is_output ? p->outputs : p->inputs; }

}  // namespace

extern "C" {

int vxb_package_open(const char* graph_path, const char* const* weight_paths, size_t weight_path_count, VxbPackage** out) {
    if (!graph_path || !out || (weight_path_count && !weight_paths)) return set_error(0, "null argument");
    *out = nullptr;
    std::unique_ptr<VxbPackage> pkg(new VxbPackage());
    pkg->files.reserve(weight_path_count + 1);
    for (size_t i = 0; i < weight_path_count; i++) {
        if (!weight_paths[i]) return set_error(0, "null weight path");
        if (load_safetensors(*pkg, weight_paths[i]) != 1) return 0;
    }
    std::vector<unsigned char> text;
    if (!read_file(graph_path, text)) return set_error(0, "cannot read %s", graph_path);
    Json graph; std::string error;
    if (!parse_json((const char*)text.data(), text.size(), graph, error) || graph.kind != Json::Object)
        return set_error(0, "%s is not a JSON object (%s)", graph_path, error.c_str());
    if (build_graph(*pkg, graph) != 1) return 0;
    *out = pkg.release();
    return 1;
}

void vxb_package_close(VxbPackage* package) { delete package; }
uint32_t vxb_package_node_count(const VxbPackage* p) { return p ? (uint32_t)p->nodes.size() : 0; }
const char* vxb_package_node_op(const VxbPackage* p, uint32_t i) { return p && i < p->nodes.size() ? p->nodes[i].op_name.c_str() : nullptr; }
uint32_t vxb_package_io_count(const VxbPackage* p, int is_output) { return p ? (uint32_t)io_list(p, is_output).size() : 0; }
const char* vxb_package_io_name(const VxbPackage* p, int is_output, uint32_t i) {
    return p && i < io_list(p, is_output).size() ? p->tensors[io_list(p, is_output)[i]].name.c_str() : nullptr;
}
uint32_t vxb_package_io_dtype(const VxbPackage* p, int is_output, uint32_t i) {
    return p && i < io_list(p, is_output).size() ? p->tensors[io_list(p, is_output)[i]].dtype : 0;
}
uint32_t vxb_package_io_rank(const VxbPackage* p, int is_output, uint32_t i) {
    return p && i < io_list(p, is_output).size() ? (uint32_t)p->tensors[io_list(p, is_output)[i]].shape.size() : 0;
}
int64_t vxb_package_io_dim(const VxbPackage* p, int is_output, uint32_t i, uint32_t axis) {
    if (!p || i >= io_list(p, is_output).size()) return 0;
    const GraphTensor& t = p->tensors[io_list(p, is_output)[i]];
    return axis < t.shape.size() ? t.shape[axis] : 0;
}
uint64_t vxb_package_io_bytes(const VxbPackage* p, int is_output, uint32_t i) {
    return p && i < io_list(p, is_output).size() ? p->tensors[io_list(p, is_output)[i]].bytes() : 0;
}

int vxb_program_compile(VxbContext* ctx, const VxbPackage* package, VxbProgram** out) {
    if (!ctx || !package || !out) return set_error(0, "null argument");
    *out = nullptr;
    std::unique_ptr<VxbProgram> prog(new VxbProgram());
    prog->ctx = ctx; prog->tensors = package->tensors; prog->inputs = package->inputs; prog->outputs = package->outputs;
    prog->nodes = package->nodes;
    prog->weights.assign(prog->nodes.size(), nullptr);
    prog->buffers.assign(prog->tensors.size(), nullptr);
    int rc = 1;
    for (size_t i = 0; rc == 1 && i < prog->nodes.size(); i++) {
        const Node& n = prog->nodes[i];
        if (n.op == kQLinear)
            rc = vxb_weight_create_i8(ctx, (const int8_t*)n.weight->data, (const float*)n.weight_scale->data, nullptr,
                                      (const int32_t*)n.bias->data, n.d_out, n.d_in, &prog->weights[i]);
        else if (n.op == kPackedLinear)
            rc = n.weight_bits == 8
                ? vxb_weight_create_w8_words(ctx, (const int32_t*)n.words->data, (const float*)n.group_scales->data,
                                             n.bias_f32 ? (const float*)n.bias_f32->data : nullptr, n.d_out, n.d_in, n.group_size, &prog->weights[i])
                : vxb_weight_create_w4_words(ctx, (const int32_t*)n.words->data, (const float*)n.group_scales->data,
                                             n.bias_f32 ? (const float*)n.bias_f32->data : nullptr, n.d_out, n.d_in, n.group_size, &prog->weights[i]);
        if (rc == 1 && prog->weights[i]) prog->device_bytes += vxb_weight_device_bytes(prog->weights[i]);
    }
    for (size_t t = 0; rc == 1 && t < prog->tensors.size(); t++) {
        if (cudaMalloc(&prog->buffers[t], prog->tensors[t].bytes()) != cudaSuccess) rc = set_error(0, "device allocation of tensor %s failed", prog->tensors[t].name.c_str());
        else prog->device_bytes += prog->tensors[t].bytes();
    }
    if (rc != 1) { vxb_program_destroy(prog.release()); return rc; }
    // the stored-tensor pointers belong to the package: the program must not follow them any more
    for (Node& n : prog->nodes) n.weight = n.weight_scale = n.bias = n.words = n.group_scales = n.bias_f32 = nullptr;
    *out = prog.release();
    return 1;
}

void vxb_program_destroy(VxbProgram* program) {
    if (!program) return;
    if (program->ctx) vxb_context_synchronize(program->ctx);
    for (VxbWeight* w : program->weights) vxb_weight_destroy(w);
    for (void* b : program->buffers) if (b) cudaFree(b);
    delete program;
}

uint64_t vxb_program_device_bytes(const VxbProgram* program) { return program ? program->device_bytes : 0; }
const char* vxb_program_route_evidence(const VxbProgram* program) { return program ? program->evidence.c_str() : ""; }

int vxb_program_execute(VxbProgram* program, const void* const* inputs, const size_t* input_bytes, uint32_t input_count,
                        void* const* outputs, const size_t* output_bytes, uint32_t output_count) {
    if (!program || !inputs || !input_bytes || !outputs || !output_bytes) return set_error(0, "null argument");
    VxbProgram& p = *program;
    // validate the complete invocation before anything is dispatched
    if (input_count != p.inputs.size() || output_count != p.outputs.size()) return set_error(0, "the package has %zu inputs and %zu outputs", p.inputs.size(), p.outputs.size());
    for (uint32_t i = 0; i < input_count; i++)
        if (!inputs[i] || input_bytes[i] != p.tensors[p.inputs[i]].bytes()) return set_error(0, "input %s needs %zu bytes", p.tensors[p.inputs[i]].name.c_str(), p.tensors[p.inputs[i]].bytes());
    for (uint32_t i = 0; i < output_count; i++)
        if (!outputs[i] || output_bytes[i] != p.tensors[p.outputs[i]].bytes()) return set_error(0, "output %s needs %zu bytes", p.tensors[p.outputs[i]].name.c_str(), p.tensors[p.outputs[i]].bytes());
    cudaStream_t stream = context_stream(p.ctx);
    for (uint32_t i = 0; i < input_count; i++)
        if (cudaMemcpyAsync(p.buffers[p.inputs[i]], inputs[i], input_bytes[i], cudaMemcpyHostToDevice, stream) != cudaSuccess)
            return set_error(-1, "input upload failed");
    p.evidence.clear();
    for (size_t i = 0; i < p.nodes.size(); i++) {
        const Node& n = p.nodes[i];
        const GraphTensor& x = p.tensors[n.input]; const GraphTensor& y = p.tensors[n.output];
        void* xin = p.buffers[n.input]; void* yout = p.buffers[n.output];
        int rc = 1;
        switch (n.op) {
            case kQuantize: rc = vxb_quantize_linear_device(p.ctx, (const float*)xin, x.elements(), n.out_q.scale, n.out_q.zero, y.dtype, yout); break;
            case kDequantize: rc = vxb_dequantize_linear_device(p.ctx, xin, x.elements(), n.in_q.scale, n.in_q.zero, x.dtype, (float*)yout); break;
            case kRequantize:
                rc = vxb_requantize_linear_device(p.ctx, xin, x.elements(), n.in_q.scale, n.in_q.zero, n.out_q.scale, n.out_q.zero, x.dtype, y.dtype, yout);
                break;
            case kQLinear:
                rc = vxb_qlinear_device(p.ctx, p.weights[i], xin, x.rows(), n.in_q.scale, n.in_q.zero, n.out_q.scale, n.out_q.zero, x.dtype, y.dtype,
                                        yout, n.d_out, VXB_ROUTE_AUTO);
                break;
            case kPackedLinear: rc = vxb_linear_f32(p.ctx, p.weights[i], (const float*)xin, x.rows(), (float*)yout, n.d_out, VXB_ROUTE_AUTO); break;
        }
        if (rc != 1) {
            // nothing of this pass reaches the caller's outputs; work of earlier nodes may be queued
            vxb_context_synchronize(p.ctx);
            return i == 0 && rc == 0 ? 0 : -1;
        }
        p.evidence += n.id + "=" + (n.op == kQLinear || n.op == kPackedLinear ? vxb_last_route() : n.op_name.c_str()) + ";";
    }
    for (uint32_t i = 0; i < output_count; i++)
        if (cudaMemcpyAsync(outputs[i], p.buffers[p.outputs[i]], output_bytes[i], cudaMemcpyDeviceToHost, stream) != cudaSuccess)
            return set_error(-1, "output download failed");
    return vxb_context_synchronize(p.ctx) == 1 ? 1 : -1;
}

}  // extern "C"
