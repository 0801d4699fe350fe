// Reverse-mode engine: graph discovery, version preflight, evaluation with a ready
// queue, staged leaf commits, hooks, finalizers and history release.
//
// Parity (reference project paths): src/autograd/engine.cpp:78-224 (GraphTask phases),
// src/autograd/node.cpp:8-43 (edge capture, saved-version text),
// src/autograd/grad_mode.cpp:5-27 (thread-local grad mode).
#include <deque>
#include <unordered_map>
#include <unordered_set>

#include "ob/ops.h"
#include "ob/tensor.h"

namespace ob {

namespace {
thread_local bool g_grad_enabled = true;
const char* kFreedGraph = "Cannot call backward twice on a freed graph. Use retain_graph=True.";
}  // namespace

bool grad_enabled() { return g_grad_enabled; }
void set_grad_enabled(bool on) { g_grad_enabled = on; }

bool needs_graph(std::initializer_list<Tensor> inputs) {
  if (!g_grad_enabled) return false;
  for (const Tensor& t : inputs)
    if (t.defined() && t.requires_grad()) return true;
  return false;
}

void attach(Tensor& out, std::shared_ptr<Node> node) {
  node->out_shape = out.shape();
  node->out_dtype = out.dtype();
  node->out_device = out.device();
  AutogradMeta& m = out.impl()->ag();
  m.requires_grad = true;
  m.grad_fn = std::move(node);
  m.history = History::Live;
}

GraphEdge GraphEdge::capture(const Tensor& t) {
  GraphEdge e;
  if (!t.defined() || !t.requires_grad()) return e;
  if (t.grad_fn()) {
    if (t.grad_fn()->released()) {
      e.kind = Released;
    } else {
      e.kind = Producer;
      e.node = t.grad_fn();
    }
  } else {
    e.kind = Leaf;
    e.leaf = t.impl();
  }
  return e;
}

void Node::set_inputs(std::initializer_list<Tensor> inputs) {
  edges_.clear();
  edges_.reserve(inputs.size());
  for (const Tensor& t : inputs) edges_.push_back(GraphEdge::capture(t));
}

void Node::set_inputs(const std::vector<Tensor>& inputs) {
  edges_.clear();
  edges_.reserve(inputs.size());
  for (const Tensor& t : inputs) edges_.push_back(GraphEdge::capture(t));
}

void Node::watch_version(const Tensor& t, const char* role) {
  saved_.push_back(SavedVersion{t.impl()->buffer(), t.version(), role});
}

void Node::validate_saved_versions() const {
  for (const SavedVersion& s : saved_) {
    const uint64_t now = s.buffer->version();
    if (now != s.version) {
      throw std::runtime_error(std::string("backward: tensor saved by ") + name() + " as '" + s.role +
                               "' was modified in-place after it was saved for backward (expected version " +
                               std::to_string(s.version) + ", found " + std::to_string(now) + ")");
    }
  }
}

void Node::mark_released() {
  released_ = true;
  release_saved();
  saved_.clear();
  for (GraphEdge& e : edges_) {
    if (e.kind != GraphEdge::None) e.kind = GraphEdge::Released;
    e.node.reset();
    e.leaf.reset();
  }
}

namespace {

struct GraphTask {
  std::vector<std::shared_ptr<Node>> nodes;  // discovery order
  std::unordered_map<Node*, int> deps;
  std::vector<std::shared_ptr<TensorImpl>> leaves;  // discovery order, unique
  std::unordered_set<TensorImpl*> leaf_set;
  std::unordered_map<TensorImpl*, int> leaf_edges;  // graph edges that still owe this leaf a gradient
  std::unordered_map<TensorImpl*, int> leaf_uses;   // graph edges that reach this leaf (fixed after discovery)
  std::vector<std::pair<uint64_t, std::function<void()>>> finalizers;
  std::unordered_set<uint64_t> finalizer_keys;

  void add_finalizers(const std::vector<std::pair<uint64_t, std::function<void()>>>& fs) {
    for (const auto& f : fs)
      if (finalizer_keys.insert(f.first).second) finalizers.push_back(f);
  }

  void add_leaf(const std::shared_ptr<TensorImpl>& leaf) {
    if (leaf_set.insert(leaf.get()).second) {
      leaves.push_back(leaf);
      add_finalizers(leaf->ag().finalizers);
    }
  }

  void discover(const std::shared_ptr<Node>& root) {
    // Iterative DFS; colour 1 = on stack, 2 = done.  A node reached while grey is a cycle.
    std::unordered_map<Node*, int> colour;
    std::vector<std::pair<std::shared_ptr<Node>, size_t>> stack;
    if (root->released()) throw std::runtime_error(kFreedGraph);
    stack.emplace_back(root, 0);
    colour[root.get()] = 1;
    nodes.push_back(root);
    deps[root.get()] = 0;
    add_finalizers(root->finalizers);
    while (!stack.empty()) {
      auto& [node, next] = stack.back();
      if (next >= node->edges().size()) {
        colour[node.get()] = 2;
        stack.pop_back();
        continue;
      }
      const GraphEdge& e = node->edges()[next++];
      if (e.kind == GraphEdge::Released) throw std::runtime_error(kFreedGraph);
      if (e.kind == GraphEdge::Leaf) {
        add_leaf(e.leaf);
        ++leaf_edges[e.leaf.get()];
        ++leaf_uses[e.leaf.get()];
      } else if (e.kind == GraphEdge::Producer) {
        if (e.node->released()) throw std::runtime_error(kFreedGraph);
        ++deps[e.node.get()];
        auto it = colour.find(e.node.get());
        if (it == colour.end()) {
          colour[e.node.get()] = 1;
          nodes.push_back(e.node);
          add_finalizers(e.node->finalizers);
          stack.emplace_back(e.node, 0);
        } else if (it->second == 1) {
          throw std::runtime_error("backward: the autograd graph contains a cycle");
        }
      }
    }
  }
};

Tensor accumulate(const Tensor& a, const Tensor& b) {
  if (!a.defined()) return b;
  return ops::add(ops::contiguous(a), ops::contiguous(b));
}

void check_grad(const Tensor& g, const Shape& shape, DType dtype, Device dev, const char* who) {
  if (g.shape() != shape)
    throw std::runtime_error(std::string("backward: ") + who + " produced a gradient of shape " +
                             shape_str(g.shape()) + ", expected " + shape_str(shape));
  if (g.dtype() != dtype)
    throw std::runtime_error(std::string("backward: ") + who + " produced a gradient of dtype " +
                             dtype_name(g.dtype()) + ", expected " + dtype_name(dtype));
  if (g.device() != dev)
    throw std::runtime_error(std::string("backward: ") + who + " produced a gradient on " + g.device().str() +
                             ", expected " + dev.str());
}

}  // namespace

void AutogradEngine::backward(const Tensor& root, bool retain_graph) {
  if (!root.defined()) throw std::invalid_argument("backward: undefined tensor");
  if (!root.requires_grad()) throw std::runtime_error("backward: tensor does not require grad");
  NoGradGuard no_grad;

  GraphTask task;
  std::unordered_map<TensorImpl*, Tensor> leaf_grads;
  Tensor seed = Tensor::full(root.shape(), 1.0, root.dtype(), root.device());

  if (root.is_leaf()) {
    task.add_leaf(root.impl());
    leaf_grads[root.raw()] = seed;
  } else {
    const std::shared_ptr<Node>& root_node = root.grad_fn();
    task.discover(root_node);
    for (const auto& n : task.nodes) n->validate_saved_versions();  // preflight

    std::unordered_map<Node*, Tensor> grads;
    grads[root_node.get()] = seed;
    std::deque<std::shared_ptr<Node>> ready;
    ready.push_back(root_node);

    // Nodes that end up with no incoming gradient still release their producers.
    std::function<void(const std::shared_ptr<Node>&)> settle = [&](const std::shared_ptr<Node>& n) {
      std::vector<std::shared_ptr<Node>> work{n};
      while (!work.empty()) {
        auto cur = work.back();
        work.pop_back();
        if (grads.count(cur.get())) {
          ready.push_back(cur);
          continue;
        }
        for (const GraphEdge& e : cur->edges())
          if (e.kind == GraphEdge::Producer && --task.deps[e.node.get()] == 0) work.push_back(e.node);
      }
    };

    while (!ready.empty()) {
      std::shared_ptr<Node> node = ready.front();
      ready.pop_front();
      Tensor g = grads[node.get()];
      grads.erase(node.get());
      node->validate_saved_versions();
      check_grad(g, node->out_shape, node->out_dtype, node->out_device, node->name());
      const auto& edges = node->edges();
      // A leaf with a preassigned gradient slot and this node as its only consumer, not
      // accumulating onto an earlier gradient: offer the slot as the formula's destination.
      bool offered = false;
      for (size_t i = 0; i < edges.size(); ++i) {
        const GraphEdge& e = edges[i];
        if (e.kind != GraphEdge::Leaf) continue;
        AutogradMeta& m = e.leaf->ag();
        if (!m.grad_slot || task.leaf_uses[e.leaf.get()] != 1) continue;
        if (m.grad && m.grad->buffer() == m.grad_slot->buffer()) continue;
        if (!offered) { node->grad_out.assign(edges.size(), Tensor()); offered = true; }
        node->grad_out[i] = Tensor(m.grad_slot);
      }
      // A producer that already holds a partial sum from its other consumers (the skip path of
      // a residual connection) and that this node reaches through one edge only: offer the sum
      // as an addend.
      bool addends = false;
      for (size_t i = 0; i < edges.size(); ++i) {
        const GraphEdge& e = edges[i];
        if (e.kind != GraphEdge::Producer) continue;
        auto it = grads.find(e.node.get());
        if (it == grads.end() || !it->second.defined()) continue;
        size_t same = 0;
        for (const GraphEdge& o : edges) same += (o.kind == GraphEdge::Producer && o.node.get() == e.node.get()) ? 1 : 0;
        if (same != 1) continue;
        if (!addends) { node->grad_addend.assign(edges.size(), Tensor()); node->addend_taken.assign(edges.size(), 0); addends = true; }
        node->grad_addend[i] = it->second;
      }
      std::vector<Tensor> in_grads;
      std::vector<char> taken;
      try {
        in_grads = node->backward(g);
      } catch (...) {
        node->grad_out.clear();
        node->grad_addend.clear();
        node->addend_taken.clear();
        throw;
      }
      if (offered) node->grad_out.clear();
      if (addends) {
        taken.swap(node->addend_taken);
        node->grad_addend.clear();
        node->addend_taken.clear();
      }
      if (in_grads.size() > edges.size())
        throw std::runtime_error(std::string("backward: ") + node->name() + " returned too many gradients");
      for (size_t i = 0; i < edges.size(); ++i) {
        const GraphEdge& e = edges[i];
        const bool has = i < in_grads.size() && in_grads[i].defined();
        if (e.kind == GraphEdge::Leaf) {
          if (has) {
            const TensorImpl& L = *e.leaf;
            check_grad(in_grads[i], L.layout().shape(), L.dtype(), L.device(), node->name());
            Tensor& slot = leaf_grads[e.leaf.get()];
            slot = accumulate(slot, in_grads[i]);
          }
          // A leaf whose gradient storage was preassigned (reducer bucket slot) is committed
          // the moment its last consumer has run, so its bucket can start reducing while the
          // rest of backward is still executing.  Such leaves give up the all-or-nothing
          // publication of the staged path below.
          if (--task.leaf_edges[e.leaf.get()] == 0 && e.leaf->ag().grad_slot) {
            auto it = leaf_grads.find(e.leaf.get());
            if (it != leaf_grads.end() && it->second.defined()) {
              AutogradMeta& m = e.leaf->ag();
              Tensor slot(m.grad_slot);
              const bool accumulating = m.grad && m.grad->buffer() == m.grad_slot->buffer();
              const bool in_place = it->second.impl()->buffer() == slot.impl()->buffer() && it->second.data() == slot.data();
              if (accumulating) ops::add_(slot, it->second, 1.0);
              else if (in_place) slot.bump_version();  // the formula wrote the slot itself
              else ops::copy_(slot, it->second);
              m.grad = m.grad_slot;
              leaf_grads.erase(it);
              auto hooks = m.post_accumulate_hooks;
              for (auto& h : hooks) h();
            }
          }
        } else if (e.kind == GraphEdge::Producer) {
          if (has) {
            check_grad(in_grads[i], e.node->out_shape, e.node->out_dtype, e.node->out_device, node->name());
            Tensor& slot = grads[e.node.get()];
            if (i < taken.size() && taken[i]) slot = in_grads[i];   // the formula already added the running sum
            else slot = accumulate(slot, in_grads[i]);
          }
          if (--task.deps[e.node.get()] == 0) settle(e.node);
        }
      }
    }
  }

  // Stage every leaf result before publishing any of them.
  struct Commit { std::shared_ptr<TensorImpl> leaf; Tensor value; bool into_slot; bool add_into_slot; };
  std::vector<Commit> commits;
  for (const auto& leaf : task.leaves) {
    auto it = leaf_grads.find(leaf.get());
    if (it == leaf_grads.end() || !it->second.defined()) continue;
    Tensor g = it->second;
    AutogradMeta& m = leaf->ag();
    if (m.grad_slot) {
      const bool accumulating = m.grad && m.grad->buffer() == m.grad_slot->buffer();
      commits.push_back({leaf, g, true, accumulating});
      continue;
    }
    if (m.grad) {
      g = ops::add(ops::contiguous(Tensor(m.grad)), ops::contiguous(g));
    } else if (!g.is_contiguous() || g.impl()->buffer().use_count() > 1 || g.impl().use_count() > 2) {
      g = ops::clone(g);  // `.grad` never aliases another tensor's storage
    }
    commits.push_back({leaf, g, false, false});
  }
  for (Commit& c : commits) {
    AutogradMeta& m = c.leaf->ag();
    if (c.into_slot) {
      Tensor slot(m.grad_slot);
      const bool in_place = c.value.impl()->buffer() == slot.impl()->buffer() && c.value.data() == slot.data();
      if (c.add_into_slot) ops::add_(slot, c.value, 1.0);
      else if (in_place) slot.bump_version();
      else ops::copy_(slot, c.value);
      m.grad = m.grad_slot;
    } else {
      m.grad = c.value.detach().impl();
    }
  }
  for (Commit& c : commits) {
    auto hooks = c.leaf->ag().post_accumulate_hooks;  // copy: a hook may register another
    for (auto& h : hooks) h();
  }
  auto finalizers = task.finalizers;
  for (auto& f : finalizers) f.second();
  if (!retain_graph) {
    for (const auto& n : task.nodes) n->mark_released();
  }
}

}  // namespace ob
