// Tensor / Node / engine with the reference's names and calling conventions
// (reference: src/engine.h), backed by device memory. See dg_runtime.h for the mirror rules.
#pragma once
#include "dg_runtime.h"

struct Tensor;
struct Node;

// Graph edge (reference: src/engine.h:22-25)
struct Edge {
  std::shared_ptr<Node> function;
  int input_slot = 0;
  Edge() = default;
  Edge(std::shared_ptr<Node> f, int slot) : function(std::move(f)), input_slot(slot) {}
};

// Backward-graph vertex and public extension point (reference: src/engine.h:28-42)
struct Node {
  std::vector<Edge> next_edges;
  virtual ~Node() = default;
  virtual std::vector<std::shared_ptr<Tensor>> apply(const std::vector<std::shared_ptr<Tensor>>& grads) = 0;
  virtual void release_variables() {}
  void add_next_edge(std::shared_ptr<Node> fn, int slot = 0) { next_edges.emplace_back(std::move(fn), slot); }
};

// Flat fp32 storage: device buffer + host mirror, each created on first use.
struct Storage {
  std::vector<float> data;   // host mirror (empty until the host touches the tensor)
  size_t n = 0;
  std::unique_ptr<dgshim::DevBuf> dev_buf;
  bool host_valid = false, dev_valid = false;  // both false = logically all zeros

  explicit Storage(size_t size) : n(size) {}

  void ensure_host() {
    if (data.size() != n) { data.assign(n, 0.0f); if (!dev_valid) host_valid = true; }
    if (!host_valid) {
      if (dev_valid) dgshim::check(dg_rt_d2h(data.data(), dev_buf->p, n * sizeof(float), dgshim::stream()), "download");
      host_valid = true;
    }
  }
  void ensure_dev() {
    if (!dev_buf) { dev_buf = std::make_unique<dgshim::DevBuf>(n * sizeof(float), !host_valid); if (!host_valid) dev_valid = true; }
    if (!dev_valid) {
      if (host_valid) dgshim::check(dg_rt_h2d(dev_buf->p, data.data(), n * sizeof(float), dgshim::stream()), "upload");
      else dgshim::check(dg_rt_memset(dev_buf->p, 0, n * sizeof(float), dgshim::stream()), "memset");
      dev_valid = true;
    }
  }
  float* host_rw() { ensure_host(); dev_valid = false; return data.data(); }
  const float* host_ro() { ensure_host(); return data.data(); }
  float* dev_rw() { ensure_dev(); host_valid = false; return static_cast<float*>(dev_buf->p); }
  const float* dev_ro() { ensure_dev(); return static_cast<const float*>(dev_buf->p); }
};

// Row-major strides (reference: src/engine.h:52-60)
inline std::vector<int> make_strides(const std::vector<int>& shape) {
  assert(!shape.empty());
  std::vector<int> s(shape.size(), 1);
  for (int i = (int)shape.size() - 2; i >= 0; --i) s[i] = s[i + 1] * shape[i + 1];
  return s;
}

// Flat index -> multi-index (reference: src/engine.h:63-73)
inline std::vector<int> unravel(int flat, const std::vector<int>& shape) {
  std::vector<int> idx(shape.size(), 0);
  for (int i = (int)shape.size() - 1; i >= 0; --i) { idx[i] = flat % shape[i]; flat /= shape[i]; }
  return idx;
}

struct Tensor : std::enable_shared_from_this<Tensor> {
  std::shared_ptr<Storage> storage;
  std::vector<int> shape, strides;
  int offset = 0;
  bool requires_grad = true;
  std::shared_ptr<Tensor> grad;
  std::shared_ptr<Node> grad_fn;
  std::shared_ptr<Node> grad_accumulator;

  Tensor(const std::vector<int>& shape_, bool req_grad = true) : shape(shape_), requires_grad(req_grad) {
    strides = make_strides(shape);
    size_t total = 1;
    for (int d : shape) total *= (size_t)d;
    storage = std::make_shared<Storage>(total);
  }

  // ---- host access (reference: src/engine.h:100-135)
  float* data_ptr() { return storage->host_rw() + offset; }
  float* grad_ptr() {
    if (!grad) grad = std::make_shared<Tensor>(shape, false);
    return grad->storage->host_rw() + grad->offset;
  }
  float data_at(int i) { return storage->host_ro()[offset + i]; }
  float grad_at(int i) { return grad ? grad->storage->host_ro()[grad->offset + i] : 0.0f; }

  // ---- device access for the ops
  const float* dev_ro() { return storage->dev_ro() + offset; }
  float* dev_rw() { return storage->dev_rw() + offset; }

  int ndim() const { return (int)shape.size(); }
  int size() const { int t = 1; for (int d : shape) t *= d; return t; }
  int flat_idx(const std::vector<int>& idx) const {
    int f = 0;
    for (size_t i = 0; i < idx.size(); ++i) f += idx[i] * strides[i];
    return f;
  }
  bool is_contiguous() const { return strides == make_strides(shape); }
  void zero_grad() { grad = nullptr; }

  // Copy a flat vector in logical order; stride-aware (reference: src/engine.h:143-154)
  void fill(const std::vector<float>& values) {
    if ((int)values.size() != size()) throw std::runtime_error("fill: value count does not match tensor size");
    float* p = storage->host_rw() + offset;
    if (is_contiguous()) { std::copy(values.begin(), values.end(), p); return; }
    for (int i = 0; i < size(); ++i) p[flat_idx(unravel(i, shape))] = values[i];
  }

  std::shared_ptr<Tensor> alias(const std::vector<int>& new_shape, const std::vector<int>& new_strides) {
    auto t = std::make_shared<Tensor>(std::vector<int>{1}, requires_grad);
    t->storage = storage;
    t->shape = new_shape;
    t->strides = new_strides;
    t->offset = offset;
    return t;
  }

  std::shared_ptr<Tensor> _view(const std::vector<int>& new_shape) {
    if (!is_contiguous()) throw std::runtime_error("view: tensor is not contiguous");
    int total = 1;
    for (int d : new_shape) total *= d;
    if (total != size()) throw std::runtime_error("view: element count differs");
    return alias(new_shape, make_strides(new_shape));
  }
  std::shared_ptr<Tensor> _reshape(const std::vector<int>& new_shape);
  std::shared_ptr<Tensor> reshape(const std::vector<int>& new_shape) { return _reshape(new_shape); }
  std::shared_ptr<Tensor> _transpose(int d0 = -2, int d1 = -1) {
    int nd = ndim();
    if (d0 < 0) d0 += nd;
    if (d1 < 0) d1 += nd;
    if (d0 < 0 || d1 < 0 || d0 >= nd || d1 >= nd) throw std::runtime_error("transpose: bad dims");
    auto sh = shape, st = strides;
    std::swap(sh[d0], sh[d1]);
    std::swap(st[d0], st[d1]);
    return alias(sh, st);
  }
  std::shared_ptr<Tensor> transpose(int d0 = -2, int d1 = -1) { return _transpose(d0, d1); }

  // Nested-bracket print, stride-aware; sub-arrays of every non-innermost dim start on a new line
  // indented by their depth, then ", shape=(a,b)" (same text as reference: src/engine.h:221-258).
  void print_rec(const float* base, int dim, int off, std::ostream& os) const {
    const bool inner = dim == ndim() - 1;
    os << "[";
    for (int i = 0; i < shape[dim]; ++i) {
      if (i > 0) os << (inner ? ", " : ",\n" + std::string(dim + 1, ' '));
      if (inner) os << (base ? base[off + i * strides[dim]] : 0.0f);
      else print_rec(base, dim + 1, off + i * strides[dim], os);
    }
    os << "]";
  }
  void show_shape(std::ostream& os) const {
    os << ", shape=(";
    for (size_t i = 0; i < shape.size(); ++i) os << shape[i] << (i + 1 < shape.size() ? "," : "");
    os << ")\n";
  }
  void show() { print_rec(storage->host_ro() + offset, 0, 0, std::cout); show_shape(std::cout); }
  // A tensor without a gradient prints zeros in its own shape, as the reference does.
  void show_grad() {
    if (!grad) { print_rec(nullptr, 0, 0, std::cout); show_shape(std::cout); return; }
    grad->show();
  }

  void backward(bool retain_graph = false);
};

#include "dg_engine_impl.h"   // accumulation, leaf sinks and Tensor::backward
