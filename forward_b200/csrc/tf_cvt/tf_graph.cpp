#include "tf_graph.h"

#include <cstdio>
#include <cstring>

FWD_TF_NAMESPACE_BEGIN

namespace {

// ---- protobuf wire format ------------------------------------------------------------------

struct Field {
  uint32_t number;
  uint32_t wire;      // 0 varint, 1 fixed64, 2 length-delimited, 5 fixed32
  uint64_t value;     // varint / fixed value
  const uint8_t* ptr; // length-delimited payload
  size_t len;
};

class Reader {
 public:
  Reader(const uint8_t* p, size_t n) : p_(p), end_(p + n) {}
  bool Done() const { return p_ >= end_; }
  bool ok() const { return ok_; }

  bool Next(Field* f) {
    if (!ok_ || p_ >= end_) return false;
    uint64_t key = 0;
    if (!Varint(&key)) return Fail();
    f->number = (uint32_t)(key >> 3);
    f->wire = (uint32_t)(key & 7);
    f->ptr = nullptr;
    f->len = 0;
    f->value = 0;
    switch (f->wire) {
      case 0:
        if (!Varint(&f->value)) return Fail();
        return true;
      case 1:
        if ((size_t)(end_ - p_) < 8) return Fail();
        std::memcpy(&f->value, p_, 8);
        p_ += 8;
        return true;
      case 5: {
        if ((size_t)(end_ - p_) < 4) return Fail();
        uint32_t v;
        std::memcpy(&v, p_, 4);
        f->value = v;
        p_ += 4;
        return true;
      }
      case 2: {
        uint64_t n = 0;
        if (!Varint(&n) || n > (uint64_t)(end_ - p_)) return Fail();
        f->ptr = p_;
        f->len = (size_t)n;
        p_ += n;
        return true;
      }
      default:
        return Fail();  // groups are not used by these messages
    }
  }

 private:
  bool Varint(uint64_t* out) {
    uint64_t r = 0;
    for (int shift = 0; shift < 64; shift += 7) {
      if (p_ >= end_) return false;
      const uint8_t c = *p_++;
      r |= (uint64_t)(c & 0x7f) << shift;
      if (!(c & 0x80)) {
        *out = r;
        return true;
      }
    }
    return false;
  }
  bool Fail() {
    ok_ = false;
    return false;
  }
  const uint8_t* p_;
  const uint8_t* end_;
  bool ok_{true};
};

std::string Str(const Field& f) { return std::string(reinterpret_cast<const char*>(f.ptr), f.len); }

// repeated scalar field: packed (wire 2) or one element per key
template <typename T, typename Decode>
bool Repeated(const Field& f, uint32_t elem_wire, std::vector<T>* out, Decode decode) {
  if (f.wire == elem_wire) {
    out->push_back(decode(f.value));
    return true;
  }
  if (f.wire != 2) return false;
  if (elem_wire == 0) {
    // a packed run of varints has no keys: read them one by one
    const uint8_t* p = f.ptr;
    const uint8_t* end = f.ptr + f.len;
    while (p < end) {
      uint64_t v = 0;
      int shift = 0;
      bool closed = false;
      while (p < end && shift < 64) {
        const uint8_t c = *p++;
        v |= (uint64_t)(c & 0x7f) << shift;
        shift += 7;
        if (!(c & 0x80)) {
          closed = true;
          break;
        }
      }
      if (!closed) return false;
      out->push_back(decode(v));
    }
    return true;
  }
  const size_t w = elem_wire == 5 ? 4 : 8;
  if (f.len % w) return false;
  for (size_t i = 0; i < f.len; i += w) {
    uint64_t v = 0;
    std::memcpy(&v, f.ptr + i, w);
    out->push_back(decode(v));
  }
  return true;
}

bool ParseShape(const Field& msg, std::vector<int64_t>* dims, bool* unknown_rank) {
  Reader r(msg.ptr, msg.len);
  Field f;
  while (r.Next(&f)) {
    if (f.number == 2 && f.wire == 2) {  // Dim
      Reader d(f.ptr, f.len);
      Field g;
      int64_t size = 0;
      while (d.Next(&g))
        if (g.number == 1 && g.wire == 0) size = (int64_t)g.value;
      if (!d.ok()) return false;
      dims->push_back(size);
    } else if (f.number == 3 && f.wire == 0) {
      *unknown_rank = f.value != 0;
    }
  }
  return r.ok();
}

bool ParseTensor(const Field& msg, std::shared_ptr<Tensor>* out, std::string* err) {
  Reader r(msg.ptr, msg.len);
  Field f;
  int dtype = TF_INVALID;
  std::vector<int64_t> dims;
  bool unknown_rank = false;
  std::vector<char> content;
  bool have_content = false;
  std::vector<float> fv;
  std::vector<double> dv;
  std::vector<int64_t> iv;  // int_val, int64_val, bool_val, half_val (bit patterns)
  while (r.Next(&f)) {
    switch (f.number) {
      case 1:
        dtype = (int)f.value;
        break;
      case 2:
        if (f.wire != 2 || !ParseShape(f, &dims, &unknown_rank)) return false;
        break;
      case 4:
        if (f.wire != 2) return false;
        content.assign(reinterpret_cast<const char*>(f.ptr), reinterpret_cast<const char*>(f.ptr) + f.len);
        have_content = true;
        break;
      case 5:
        if (!Repeated<float>(f, 5, &fv, [](uint64_t v) {
              uint32_t b = (uint32_t)v;
              float x;
              std::memcpy(&x, &b, 4);
              return x;
            }))
          return false;
        break;
      case 6:
        if (!Repeated<double>(f, 1, &dv, [](uint64_t v) {
              double x;
              std::memcpy(&x, &v, 8);
              return x;
            }))
          return false;
        break;
      case 7:
      case 10:
      case 11:
      case 13:
        if (!Repeated<int64_t>(f, 0, &iv, [](uint64_t v) { return (int64_t)v; })) return false;
        break;
      default:
        break;
    }
  }
  if (!r.ok()) return false;
  const size_t es = DataTypeSize(dtype);
  if (!es) {
    *err = "tensor of unsupported dtype " + std::to_string(dtype);
    *out = std::make_shared<Tensor>();  // kept as an invalid tensor: other nodes may still parse
    return true;
  }
  int64_t count = 1;
  for (int64_t d : dims) {
    if (d < 0 || (d > 0 && count > (int64_t)1 << 40)) return false;
    count *= d;
  }
  std::vector<char> bytes;
  if (have_content) {
    if ((int64_t)content.size() != count * (int64_t)es) return false;
    bytes.swap(content);
  } else {
    // typed value lists: fewer values than elements means "repeat the last one"
    bytes.resize((size_t)count * es);
    auto put = [&](int64_t i, double as_double, int64_t as_int, float as_float) {
      char* dst = bytes.data() + (size_t)i * es;
      switch (dtype) {
        case TF_FLOAT: std::memcpy(dst, &as_float, 4); break;
        case TF_DOUBLE: std::memcpy(dst, &as_double, 8); break;
        case TF_INT32: { int32_t v = (int32_t)as_int; std::memcpy(dst, &v, 4); break; }
        case TF_INT64: std::memcpy(dst, &as_int, 8); break;
        case TF_BOOL: { uint8_t v = as_int != 0; std::memcpy(dst, &v, 1); break; }
        case TF_HALF: { uint16_t v = (uint16_t)as_int; std::memcpy(dst, &v, 2); break; }
        default: break;
      }
    };
    for (int64_t i = 0; i < count; ++i) {
      if (dtype == TF_FLOAT) {
        const float v = fv.empty() ? 0.0f : fv[(size_t)i < fv.size() ? (size_t)i : fv.size() - 1];
        put(i, 0, 0, v);
      } else if (dtype == TF_DOUBLE) {
        const double v = dv.empty() ? 0.0 : dv[(size_t)i < dv.size() ? (size_t)i : dv.size() - 1];
        put(i, v, 0, 0);
      } else {
        const int64_t v = iv.empty() ? 0 : iv[(size_t)i < iv.size() ? (size_t)i : iv.size() - 1];
        put(i, 0, v, 0);
      }
    }
  }
  *out = std::make_shared<Tensor>(dtype, dims, std::move(bytes));
  return true;
}

bool ParseAttrValue(const Field& msg, AttrValue* a, std::string* err) {
  Reader r(msg.ptr, msg.len);
  Field f;
  while (r.Next(&f)) {
    switch (f.number) {
      case 1: a->kind = AttrValue::kList; break;  // lists are not needed on this path
      case 2: a->kind = AttrValue::kString; a->s = Str(f); break;
      case 3: a->kind = AttrValue::kInt; a->i = (int64_t)f.value; break;
      case 4: {
        a->kind = AttrValue::kFloat;
        uint32_t b = (uint32_t)f.value;
        std::memcpy(&a->f, &b, 4);
        break;
      }
      case 5: a->kind = AttrValue::kBool; a->b = f.value != 0; break;
      case 6: a->kind = AttrValue::kType; a->type = (int)f.value; break;
      case 7:
        a->kind = AttrValue::kShape;
        if (f.wire != 2 || !ParseShape(f, &a->shape, &a->unknown_rank)) return false;
        break;
      case 8:
        a->kind = AttrValue::kTensor;
        if (f.wire != 2 || !ParseTensor(f, &a->tensor, err)) return false;
        break;
      default: break;
    }
  }
  return r.ok();
}

bool ParseNode(const Field& msg, NodeDef* n, std::string* err) {
  Reader r(msg.ptr, msg.len);
  Field f;
  while (r.Next(&f)) {
    if (f.wire != 2) continue;
    switch (f.number) {
      case 1: n->name = Str(f); break;
      case 2: n->op = Str(f); break;
      case 3: {
        std::string in = Str(f);
        if (!in.empty() && in[0] == '^') {
          n->control_inputs.push_back(in.substr(1));
          break;
        }
        int index = 0;
        const size_t colon = in.rfind(':');
        if (colon != std::string::npos) {
          index = std::atoi(in.c_str() + colon + 1);
          in.resize(colon);
        }
        n->inputs.emplace_back(in, index);
        break;
      }
      case 4: n->device = Str(f); break;
      case 5: {  // map entry: key(1), value(2)
        Reader e(f.ptr, f.len);
        Field g;
        std::string key;
        AttrValue value;
        while (e.Next(&g)) {
          if (g.number == 1 && g.wire == 2) key = Str(g);
          if (g.number == 2 && g.wire == 2 && !ParseAttrValue(g, &value, err)) return false;
        }
        if (!e.ok()) return false;
        n->attrs[key] = std::move(value);
        break;
      }
      default: break;
    }
  }
  return r.ok();
}

}  // namespace

size_t DataTypeSize(int dtype) {
  switch (dtype) {
    case TF_FLOAT: case TF_INT32: return 4;
    case TF_DOUBLE: case TF_INT64: return 8;
    case TF_HALF: return 2;
    case TF_BOOL: return 1;
    default: return 0;
  }
}

int Tensor::AsInt(bool* ok) const {
  const bool good = dtype_ == TF_INT32 && Size() == 1;
  if (ok) *ok = good;
  return good ? *Data<int32_t>() : 0;
}

std::vector<int> Tensor::AsIntList(bool* ok) const {
  const bool good = dtype_ == TF_INT32;
  if (ok) *ok = good;
  if (!good) return {};
  return std::vector<int>(Data<int32_t>(), Data<int32_t>() + Size());
}

bool Graph::Load(const std::string& path) {
  FILE* fp = std::fopen(path.c_str(), "rb");
  if (!fp) {
    error_ = "cannot open " + path;
    return false;
  }
  std::vector<char> bytes;
  char buf[1 << 16];
  size_t n;
  while ((n = std::fread(buf, 1, sizeof(buf), fp)) > 0) bytes.insert(bytes.end(), buf, buf + n);
  std::fclose(fp);
  return Parse(bytes.data(), bytes.size());
}

bool Graph::Parse(const void* bytes, size_t len) {
  nodes_.clear();
  by_name_.clear();
  error_.clear();
  Reader r(static_cast<const uint8_t*>(bytes), len);
  Field f;
  std::string note;
  while (r.Next(&f)) {
    if (f.number != 1 || f.wire != 2) continue;  // versions, library: not needed
    NodeDef n;
    if (!ParseNode(f, &n, &note)) {
      error_ = "malformed NodeDef (node " + std::to_string(nodes_.size()) + ")";
      nodes_.clear();
      return false;
    }
    nodes_.push_back(std::move(n));
  }
  if (!r.ok()) {
    error_ = "malformed GraphDef";
    nodes_.clear();
    return false;
  }
  if (nodes_.empty()) {
    error_ = "the GraphDef holds no nodes";
    return false;
  }
  for (size_t i = 0; i < nodes_.size(); ++i) by_name_[nodes_[i].name] = i;
  return true;
}

const NodeDef* Graph::OperationByName(const std::string& name) const {
  auto it = by_name_.find(name);
  return it == by_name_.end() ? nullptr : &nodes_[it->second];
}

Output Operation::Input(int index) const {
  if (!Valid() || index < 0 || index >= (int)node_->inputs.size()) return Output();
  const auto& in = node_->inputs[index];
  return Output(graph_, graph_->OperationByName(in.first), in.second);
}

const AttrValue* Operation::Attr(const char* name) const {
  if (!node_) return nullptr;
  auto it = node_->attrs.find(name);
  return it == node_->attrs.end() ? nullptr : &it->second;
}

bool Operation::GetAttrBool(const char* name, bool fallback) const {
  const AttrValue* a = Attr(name);
  return a && a->kind == AttrValue::kBool ? a->b : fallback;
}

int64_t Operation::GetAttrInt(const char* name, int64_t fallback) const {
  const AttrValue* a = Attr(name);
  return a && a->kind == AttrValue::kInt ? a->i : fallback;
}

int Operation::GetAttrType(const char* name) const {
  const AttrValue* a = Attr(name);
  return a && a->kind == AttrValue::kType ? a->type : TF_INVALID;
}

Tensor Output::GetConstantTensor() const {
  Output cur = *this;
  for (int hops = 0; hops < 64 && cur.Valid(); ++hops) {
    if (cur.OpType() == "Const") {
      const AttrValue* v = cur.Attr("value");
      return (v && v->kind == AttrValue::kTensor && v->tensor) ? *v->tensor : Tensor();
    }
    if (cur.OpType() != "Identity") break;
    cur = cur.Input(0);
  }
  return Tensor();
}

bool Output::GetTensorShape(std::vector<int64_t>* dims) const {
  Output cur = *this;
  for (int hops = 0; hops < 64 && cur.Valid(); ++hops) {
    if (cur.OpType() == "Const") {
      Tensor t = cur.GetConstantTensor();
      if (!t.Valid()) return false;
      *dims = t.Dims();
      return true;
    }
    if (cur.OpType() == "Placeholder") {
      const AttrValue* s = cur.Attr("shape");
      if (!s || s->kind != AttrValue::kShape || s->unknown_rank) return false;
      *dims = s->shape;
      return true;
    }
    if (cur.OpType() != "Identity") break;
    cur = cur.Input(0);
  }
  return false;
}

FWD_TF_NAMESPACE_END
