#include "dlx.h"

#include <cstdio>
#include <cstring>
#include <stdexcept>

namespace dlxnet {
namespace {

struct Malformed : std::runtime_error {
    explicit Malformed(const char* m) : std::runtime_error(m) {}
};

// Cursor over one length-delimited region of the wire.
class Reader {
public:
    Reader(const uint8_t* p, size_t n) : p_(p), end_(p + n) {}
    bool done() const { return p_ >= end_; }
    uint64_t varint() {
        uint64_t v = 0;
        for (int shift = 0; shift < 64; shift += 7) {
            if (p_ >= end_) throw Malformed("truncated varint");
            const uint8_t b = *p_++;
            v |= uint64_t(b & 0x7f) << shift;
            if (!(b & 0x80)) return v;
        }
        throw Malformed("varint too long");
    }
    uint32_t fixed32() {
        if (end_ - p_ < 4) throw Malformed("truncated fixed32");
        uint32_t v;
        std::memcpy(&v, p_, 4);
        p_ += 4;
        return v;
    }
    float f32() {
        const uint32_t u = fixed32();
        float f;
        std::memcpy(&f, &u, 4);
        return f;
    }
    Reader sub() {
        const uint64_t n = varint();
        if (n > uint64_t(end_ - p_)) throw Malformed("length-delimited field overruns its parent");
        Reader r(p_, size_t(n));
        p_ += n;
        return r;
    }
    std::string str() {
        Reader r = sub();
        return std::string(reinterpret_cast<const char*>(r.p_), size_t(r.end_ - r.p_));
    }
    void skip(int wire) {
        switch (wire) {
            case 0: varint(); break;
            case 1: if (end_ - p_ < 8) throw Malformed("truncated fixed64"); p_ += 8; break;
            case 2: sub(); break;
            case 5: fixed32(); break;
            default: throw Malformed("unsupported wire type");
        }
    }
    size_t remaining() const { return size_t(end_ - p_); }
    const uint8_t* ptr() const { return p_; }

private:
    const uint8_t* p_;
    const uint8_t* end_;
};

// repeated integer field: packed (wire 2) or one element per tag (wire 0)
template <class T>
void read_ints(Reader& r, int wire, std::vector<T>* out) {
    if (wire == 2) {
        Reader s = r.sub();
        while (!s.done()) out->push_back(T(int64_t(s.varint())));
    } else if (wire == 0) {
        out->push_back(T(int64_t(r.varint())));
    } else {
        throw Malformed("bad wire type for an integer field");
    }
}

void read_floats(Reader& r, int wire, std::vector<float>* out) {
    if (wire == 2) {
        Reader s = r.sub();
        if (s.remaining() % 4) throw Malformed("packed float field is not a multiple of 4 bytes");
        const size_t n = s.remaining() / 4;
        const size_t old = out->size();
        out->resize(old + n);
        std::memcpy(out->data() + old, s.ptr(), n * 4);
    } else if (wire == 5) {
        out->push_back(r.f32());
    } else {
        throw Malformed("bad wire type for a float field");
    }
}

float read_float(Reader& r, int wire) {
    if (wire != 5) throw Malformed("bad wire type for a float field");
    return r.f32();
}
int64_t read_int(Reader& r, int wire) {
    if (wire != 0) throw Malformed("bad wire type for an integer field");
    return int64_t(r.varint());
}

template <class F>
void for_fields(Reader r, F f) {
    while (!r.done()) {
        const uint64_t tag = r.varint();
        const int field = int(tag >> 3), wire = int(tag & 7);
        if (!f(field, wire, r)) r.skip(wire);
    }
}

void parse(Reader r, TensorProto* t) {
    for_fields(r, [&](int f, int w, Reader& s) {
        switch (f) {
            case 1: t->data_format = TensorProto::DataFormat(read_int(s, w)); return true;
            case 2: t->data_type = TensorProto::DataType(read_int(s, w)); return true;
            case 3: read_ints(s, w, &t->dims); return true;
            case 4: read_floats(s, w, &t->float_data); return true;
            case 5: read_ints(s, w, &t->int32_data); return true;
            case 7: read_ints(s, w, &t->int64_data); return true;
            case 8: t->target_data_format = TensorProto::DataFormat(read_int(s, w)); return true;
        }
        return false;
    });
}

void parse(Reader r, Conv2dAttribute* a) {
    for_fields(r, [&](int f, int w, Reader& s) {
        switch (f) {
            case 1: read_ints(s, w, &a->kernel_shape); return true;
            case 2: read_ints(s, w, &a->strides); return true;
            case 3: read_ints(s, w, &a->pads); return true;
            case 4: read_ints(s, w, &a->dilations); return true;
            case 5: a->group = read_int(s, w); return true;
            case 6: a->activation_type = s.str(); return true;
            case 7: a->min = read_float(s, w); return true;
            case 8: a->max = read_float(s, w); return true;
        }
        return false;
    });
}

template <class P>
void parse_pool(Reader r, P* a) {
    for_fields(r, [&](int f, int w, Reader& s) {
        switch (f) {
            case 1: read_ints(s, w, &a->kernel_shape); return true;
            case 2: read_ints(s, w, &a->strides); return true;
            case 3: read_ints(s, w, &a->pads); return true;
        }
        return false;
    });
}

void parse(Reader r, Attribute* a) {
    for_fields(r, [&](int f, int w, Reader& s) {
        if (w != 2) return false;
        switch (f) {
            case 1: parse(s.sub(), &a->conv2d_attr); return true;
            case 2:
                for_fields(s.sub(), [&](int f2, int w2, Reader& s2) {
                    if (f2 == 1 && w2 == 2) { parse(s2.sub(), &a->const_attr.value); return true; }
                    return false;
                });
                return true;
            case 3:
                for_fields(s.sub(), [&](int f2, int w2, Reader& s2) {
                    if (f2 == 1) { a->batchnorm_attr.momentum = read_float(s2, w2); return true; }
                    if (f2 == 2) { a->batchnorm_attr.epsilon = read_float(s2, w2); return true; }
                    return false;
                });
                return true;
            case 4:
                for_fields(s.sub(), [&](int f2, int w2, Reader& s2) {
                    if (f2 == 1) { a->relu_attr.slope = read_float(s2, w2); return true; }
                    return false;
                });
                return true;
            case 5: parse_pool(s.sub(), &a->maxpool_attr); return true;
            case 6: parse_pool(s.sub(), &a->avepool_attr); return true;
            case 7:
                for_fields(s.sub(), [&](int f2, int w2, Reader& s2) {
                    if (f2 == 1) { a->flatten_attr.axis = int32_t(read_int(s2, w2)); return true; }
                    return false;
                });
                return true;
            case 8:
                for_fields(s.sub(), [&](int f2, int w2, Reader& s2) {
                    if (f2 == 1 && w2 == 2) { a->binary_attr.binary_op_type = s2.str(); return true; }
                    return false;
                });
                return true;
            case 9:
                for_fields(s.sub(), [&](int f2, int w2, Reader& s2) {
                    if (f2 == 1) { a->gemm_attr.alpha = read_float(s2, w2); return true; }
                    if (f2 == 2) { a->gemm_attr.beta = read_float(s2, w2); return true; }
                    if (f2 == 3) { a->gemm_attr.transb = int32_t(read_int(s2, w2)); return true; }
                    return false;
                });
                return true;
            case 10:
                for_fields(s.sub(), [&](int f2, int w2, Reader& s2) {
                    if (f2 == 3) { read_ints(s2, w2, &a->input_attr.dims); return true; }
                    return false;
                });
                return true;
            case 11:
                for_fields(s.sub(), [&](int f2, int w2, Reader& s2) {
                    if (f2 == 1) { a->clip_attr.min = read_float(s2, w2); return true; }
                    if (f2 == 2) { a->clip_attr.max = read_float(s2, w2); return true; }
                    return false;
                });
                return true;
            case 12:
                for_fields(s.sub(), [&](int f2, int w2, Reader& s2) {
                    if (f2 == 1) { read_ints(s2, w2, &a->transpose_attr.perm); return true; }
                    return false;
                });
                return true;
            case 14:
                for_fields(s.sub(), [&](int f2, int w2, Reader& s2) {
                    if (f2 == 1) { a->gather_attr.axis = int32_t(read_int(s2, w2)); return true; }
                    return false;
                });
                return true;
            case 15:
                for_fields(s.sub(), [&](int f2, int w2, Reader& s2) {
                    if (f2 == 1) { read_ints(s2, w2, &a->unsqueeze_attr.axes); return true; }
                    return false;
                });
                return true;
            case 16:
                for_fields(s.sub(), [&](int f2, int w2, Reader& s2) {
                    if (f2 == 1) { a->concat_attr.axis = int32_t(read_int(s2, w2)); return true; }
                    return false;
                });
                return true;
            case 17:
                for_fields(s.sub(), [&](int f2, int w2, Reader& s2) {
                    if (f2 == 1) { a->reshape_attr.axis = int32_t(read_int(s2, w2)); return true; }
                    return false;
                });
                return true;
        }
        return false;
    });
}

void parse(Reader r, NodeProto* n) {
    for_fields(r, [&](int f, int w, Reader& s) {
        switch (f) {
            case 1: read_ints(s, w, &n->input_index); return true;
            case 2: read_ints(s, w, &n->output_index); return true;
            case 3: if (w != 2) return false; parse(s.sub(), &n->attr); return true;
            case 4: if (w != 2) return false; n->doc_string = s.str(); return true;
            case 5: if (w != 2) return false; n->name = s.str(); return true;
            case 6: if (w != 2) return false; n->type = s.str(); return true;
        }
        return false;
    });
}

void parse(Reader r, GraphProto* g) {
    for_fields(r, [&](int f, int w, Reader& s) {
        if (w != 2) return false;
        switch (f) {
            case 1: g->node.emplace_back(); parse(s.sub(), &g->node.back()); return true;
            case 2: g->name = s.str(); return true;
            case 3: g->tensor_names.push_back(s.str()); return true;
            case 4: g->output_names.push_back(s.str()); return true;
            case 5: g->input_names.push_back(s.str()); return true;
        }
        return false;
    });
}

// ------------------------------------------------------------------ writer
class Writer {
public:
    std::string out;
    void varint(uint64_t v) {
        while (v >= 0x80) { out.push_back(char(uint8_t(v) | 0x80)); v >>= 7; }
        out.push_back(char(uint8_t(v)));
    }
    void tag(int field, int wire) { varint(uint64_t(field) << 3 | uint64_t(wire)); }
    void bytes(int field, const std::string& s) { tag(field, 2); varint(s.size()); out += s; }
    void str(int field, const std::string& s) { if (!s.empty()) bytes(field, s); }
    void i64(int field, int64_t v) { if (v != 0) { tag(field, 0); varint(uint64_t(v)); } }
    void f32(int field, float v) {
        uint32_t u;
        std::memcpy(&u, &v, 4);
        if (u != 0) { tag(field, 5); out.append(reinterpret_cast<const char*>(&u), 4); }
    }
    template <class T>
    void ints(int field, const std::vector<T>& v) {
        if (v.empty()) return;
        Writer w;
        for (T x : v) w.varint(uint64_t(int64_t(x)));
        bytes(field, w.out);
    }
    void floats(int field, const std::vector<float>& v) {
        if (v.empty()) return;
        tag(field, 2);
        varint(v.size() * 4);
        out.append(reinterpret_cast<const char*>(v.data()), v.size() * 4);
    }
};

std::string ser(const TensorProto& t) {
    Writer w;
    w.i64(1, t.data_format);
    w.i64(2, t.data_type);
    w.ints(3, t.dims);
    w.floats(4, t.float_data);
    w.ints(5, t.int32_data);
    w.ints(7, t.int64_data);
    w.i64(8, t.target_data_format);
    return w.out;
}

template <class P>
std::string ser_pool(const P& a) {
    Writer w;
    w.ints(1, a.kernel_shape); w.ints(2, a.strides); w.ints(3, a.pads);
    return w.out;
}

// A sub-message is written when it differs from its default; `force` writes it
// even when empty (a present-but-empty message, e.g. Relu's attribute).
void sub(Writer& w, int field, const std::string& body) { if (!body.empty()) w.bytes(field, body); }

std::string ser(const Attribute& a, const std::string& node_type) {
    Writer w;
    {
        Writer c;
        c.ints(1, a.conv2d_attr.kernel_shape); c.ints(2, a.conv2d_attr.strides); c.ints(3, a.conv2d_attr.pads);
        c.ints(4, a.conv2d_attr.dilations); c.i64(5, a.conv2d_attr.group); c.str(6, a.conv2d_attr.activation_type);
        c.f32(7, a.conv2d_attr.min); c.f32(8, a.conv2d_attr.max);
        sub(w, 1, c.out);
    }
    if (node_type == "Const" || node_type == "Constant") {
        Writer c;
        c.bytes(1, ser(a.const_attr.value));
        w.bytes(2, c.out);
    }
    { Writer c; c.f32(1, a.batchnorm_attr.momentum); c.f32(2, a.batchnorm_attr.epsilon); sub(w, 3, c.out); }
    { Writer c; c.f32(1, a.relu_attr.slope); sub(w, 4, c.out); }
    sub(w, 5, ser_pool(a.maxpool_attr));
    sub(w, 6, ser_pool(a.avepool_attr));
    { Writer c; c.i64(1, a.flatten_attr.axis); sub(w, 7, c.out); }
    { Writer c; c.str(1, a.binary_attr.binary_op_type); sub(w, 8, c.out); }
    { Writer c; c.f32(1, a.gemm_attr.alpha); c.f32(2, a.gemm_attr.beta); c.i64(3, a.gemm_attr.transb); sub(w, 9, c.out); }
    { Writer c; c.ints(3, a.input_attr.dims); sub(w, 10, c.out); }
    { Writer c; c.f32(1, a.clip_attr.min); c.f32(2, a.clip_attr.max); sub(w, 11, c.out); }
    { Writer c; c.ints(1, a.transpose_attr.perm); sub(w, 12, c.out); }
    { Writer c; c.i64(1, a.gather_attr.axis); sub(w, 14, c.out); }
    { Writer c; c.ints(1, a.unsqueeze_attr.axes); sub(w, 15, c.out); }
    { Writer c; c.i64(1, a.concat_attr.axis); sub(w, 16, c.out); }
    { Writer c; c.i64(1, a.reshape_attr.axis); sub(w, 17, c.out); }
    return w.out;
}

}  // namespace

bool ParseModel(const void* data, size_t size, ModelProto* model, std::string* error) {
    *model = ModelProto();
    try {
        Reader r(static_cast<const uint8_t*>(data), size);
        for_fields(r, [&](int f, int w, Reader& s) {
            if (w != 2) return false;
            switch (f) {
                case 1: parse(s.sub(), &model->graph); return true;
                case 2: model->version = s.str(); return true;
                case 3: model->producer_name = s.str(); return true;
                case 4: model->doc_string = s.str(); return true;
            }
            return false;
        });
    } catch (const Malformed& e) {
        if (error) *error = e.what();
        return false;
    }
    return true;
}

bool ReadModelFromFile(const std::string& path, ModelProto* model, std::string* error) {
    FILE* f = std::fopen(path.c_str(), "rb");
    if (!f) {
        if (error) *error = "cannot open " + path;
        return false;
    }
    std::string buf;
    char chunk[1 << 16];
    size_t n;
    while ((n = std::fread(chunk, 1, sizeof(chunk), f)) > 0) buf.append(chunk, n);
    std::fclose(f);
    return ParseModel(buf.data(), buf.size(), model, error);
}

std::string SerializeModel(const ModelProto& m) {
    Writer g;
    for (const NodeProto& n : m.graph.node) {
        Writer w;
        w.ints(1, n.input_index);
        w.ints(2, n.output_index);
        const std::string a = ser(n.attr, n.type);
        if (!a.empty()) w.bytes(3, a);
        w.str(4, n.doc_string);
        w.str(5, n.name);
        w.str(6, n.type);
        g.bytes(1, w.out);
    }
    g.str(2, m.graph.name);
    for (const std::string& s : m.graph.tensor_names) g.bytes(3, s);
    for (const std::string& s : m.graph.output_names) g.bytes(4, s);
    for (const std::string& s : m.graph.input_names) g.bytes(5, s);
    Writer w;
    w.bytes(1, g.out);
    w.str(2, m.version);
    w.str(3, m.producer_name);
    w.str(4, m.doc_string);
    return w.out;
}

}  // namespace dlxnet
