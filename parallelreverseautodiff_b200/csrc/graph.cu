// Graph mode: a static-schedule backward over an operation DAG, replacing the managed
// visitor's tasks, locks and semaphores (OperationNeuralNetworkVisitor.cs:143-337) by one
// reverse walk on a stream.  Host-side C++ only; every arithmetic step is a call to one of the
// library's own entry points.
#include <algorithm>
#include <memory>

#include "common.cuh"

namespace prad {

struct GValue {
  int rows = 0, cols = 0;
  int depth = 1;               // DeepMatrix: `depth` consecutive rows x cols slices
  int64_t count() const { return (int64_t)depth * rows * cols; }
  int64_t slice() const { return (int64_t)rows * cols; }
  void* data = nullptr;        // caller-owned or graph-owned
  bool owned = false;
  void* grad_dst = nullptr;    // weight-style destination (+=)
  void* grad = nullptr;        // gradient after the last backward (may alias a contribution)
  std::vector<void*> contrib;  // contributions of the consumers, in consumer order
  void* sum_buf = nullptr;     // fan-in sum (graph-owned, reused)
  int consumers = 0;
  int produced_by = -1;        // node that writes this value (-1: a leaf holding caller data)
};

struct GNode {
  prad_op op;
  std::vector<int> in;
  int out = -1;
  double scalar = 0.0;
  // per-node state kept between forward and backward
  void* aux0 = nullptr;        // LayerNorm mean; batch product with a shared first operand: per-slice products
  void* aux1 = nullptr;        // LayerNorm sigma
  std::vector<void*> in_grad;  // gradient buffers of the inputs (graph-owned, reused)
};

}  // namespace prad

struct prad_graph {
  prad_ctx* ctx = nullptr;
  prad_dtype dt = PRAD_F32;
  std::vector<prad::GValue> values;
  std::vector<prad::GNode> nodes;
  std::vector<void*> owned;    // every device block the graph allocated
  uint32_t magic = 0x47524146u;
};

namespace prad {

static bool graph_ok(const prad_graph* g) { return g && g->magic == 0x47524146u && ctx_ok(g->ctx); }

#define PRAD_CHECK_GRAPH(g)                                                          \
  do {                                                                               \
    if (!prad::graph_ok(g)) {                                                        \
      prad::set_error("graph handle is null, destroyed, or its context was shut down"); \
      return PRAD_ERR_NOT_INITIALIZED;                                               \
    }                                                                                \
  } while (0)

static prad_status g_alloc(prad_graph* g, size_t elems, void** out) {
  prad_status s = prad_alloc(g->ctx, elems * dtype_size(g->dt), out);
  if (s == PRAD_OK) g->owned.push_back(*out);
  return s;
}

static int arity(prad_op op) {
  switch (op) {
    case PRAD_OP_MATMUL: case PRAD_OP_ADD: case PRAD_OP_ADD_BROADCAST: case PRAD_OP_HADAMARD: return 2;
    case PRAD_OP_ADD3: return 3;
    default: return 1;
  }
}

static prad_act act_of(prad_op op) {
  switch (op) {
    case PRAD_OP_LEAKY_RELU: return PRAD_ACT_LEAKY_RELU;
    case PRAD_OP_SIGMOID: return PRAD_ACT_SIGMOID;
    case PRAD_OP_TANH: return PRAD_ACT_TANH;
    case PRAD_OP_GELU: return PRAD_ACT_GELU;
    case PRAD_OP_RELU: return PRAD_ACT_RELU;
    case PRAD_OP_AMPLIFIED_SIGMOID: return PRAD_ACT_AMPLIFIED_SIGMOID;
    default: return PRAD_ACT_NONE;
  }
}

}  // namespace prad

using namespace prad;

extern "C" {

prad_status prad_graph_create(prad_ctx* ctx, prad_dtype dt, prad_graph** out_graph) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(out_graph && dtype_ok(dt), PRAD_ERR_INVALID, "prad_graph_create: bad argument");
  prad_graph* g = new prad_graph();
  g->ctx = ctx;
  g->dt = dt;
  *out_graph = g;
  return PRAD_OK;
}

prad_status prad_graph_destroy(prad_graph* g) {
  PRAD_CHECK_GRAPH(g);
  for (void* p : g->owned) prad_free(g->ctx, p);
  g->magic = 0;
  delete g;
  return PRAD_OK;
}

prad_status prad_graph_add_value(prad_graph* g, int rows, int cols, void* data, int* out_value) {
  PRAD_CHECK_GRAPH(g);
  PRAD_REQUIRE(rows > 0 && cols > 0 && out_value, PRAD_ERR_SHAPE, "prad_graph_add_value: bad shape or null output");
  GValue v;
  v.rows = rows;
  v.cols = cols;
  v.data = data;
  g->values.push_back(v);
  *out_value = (int)g->values.size() - 1;
  return PRAD_OK;
}

prad_status prad_graph_add_deep_value(prad_graph* g, int depth, int rows, int cols, void* data, int* out_value) {
  PRAD_CHECK_GRAPH(g);
  PRAD_REQUIRE(depth > 0, PRAD_ERR_SHAPE, "prad_graph_add_deep_value: depth must be positive");
  prad_status s = prad_graph_add_value(g, rows, cols, data, out_value);
  if (s == PRAD_OK) g->values[*out_value].depth = depth;
  return s;
}

prad_status prad_graph_set_gradient_destination(prad_graph* g, int value, void* grad_matrix) {
  PRAD_CHECK_GRAPH(g);
  PRAD_REQUIRE(value >= 0 && value < (int)g->values.size() && grad_matrix, PRAD_ERR_INVALID,
               "prad_graph_set_gradient_destination: bad value id or null matrix");
  g->values[value].grad_dst = grad_matrix;
  return PRAD_OK;
}

prad_status prad_graph_add_node(prad_graph* g, prad_op op, const int* in_values, int n_in,
                                int out_value, double scalar, int* out_node) {
  PRAD_CHECK_GRAPH(g);
  PRAD_REQUIRE(op >= PRAD_OP_MATMUL && op <= PRAD_OP_SINE_SOFTMAX && in_values, PRAD_ERR_INVALID,
               "prad_graph_add_node: unknown operation or null inputs");
  PRAD_REQUIRE(n_in == arity(op), PRAD_ERR_INVALID, "prad_graph_add_node: operation %d takes %d inputs, got %d",
               (int)op, arity(op), n_in);
  const int nv = (int)g->values.size();
  PRAD_REQUIRE(out_value >= 0 && out_value < nv, PRAD_ERR_INVALID, "prad_graph_add_node: bad output value id");
  for (int i = 0; i < n_in; ++i) {
    PRAD_REQUIRE(in_values[i] >= 0 && in_values[i] < nv && in_values[i] != out_value, PRAD_ERR_INVALID,
                 "prad_graph_add_node: bad input value id at position %d", i);
    // nodes arrive in forward order: an input is caller data or the output of an earlier node
    const GValue& iv = g->values[in_values[i]];
    PRAD_REQUIRE(iv.produced_by >= 0 || (iv.data != nullptr && !iv.owned), PRAD_ERR_INVALID,
                 "prad_graph_add_node: input %d (value %d) has neither caller data nor an earlier producer", i,
                 in_values[i]);
  }
  GValue& o = g->values[out_value];
  PRAD_REQUIRE(o.data == nullptr || o.owned, PRAD_ERR_INVALID,
               "prad_graph_add_node: the output value must be graph-owned (added with data == NULL)");
  PRAD_REQUIRE(o.produced_by < 0, PRAD_ERR_INVALID,
               "prad_graph_add_node: value %d is already the output of node %d", out_value, o.produced_by);
  auto& V = g->values;
  const GValue& a = V[in_values[0]];
  // Batch* operations: the output is a DeepMatrix of D slices; every input has D slices, or is one Matrix
  // shared by all slices (BatchMatrixAddOperation.Forward(DeepMatrix, Matrix), BatchGpuMatrixMultiplyOperation
  // .Forward(Matrix, DeepMatrix) ...).  A shared input must be a leaf: its gradient is the visitor's mean
  // over the slices (OperationNeuralNetworkVisitor.cs:449-478), which only a destination can receive.
  const int D = o.depth;
  for (int i = 0; i < n_in; ++i) {
    const GValue& iv = V[in_values[i]];
    PRAD_REQUIRE(iv.depth == D || iv.depth == 1, PRAD_ERR_SHAPE,
                 "prad_graph_add_node: input %d has %d slices, the output %d", i, iv.depth, D);
    if (D > 1 && iv.depth == 1) {
      const bool may_share = op == PRAD_OP_MATMUL || (op == PRAD_OP_ADD && i == 1) || (op == PRAD_OP_ADD3 && i == 2) ||
                             (op == PRAD_OP_ADD_BROADCAST && i == 1);
      PRAD_REQUIRE(may_share, PRAD_ERR_SHAPE, "prad_graph_add_node: input %d of operation %d cannot be shared by the slices", i,
                   (int)op);
      PRAD_REQUIRE(iv.produced_by < 0, PRAD_ERR_UNSUPPORTED,
                   "prad_graph_add_node: a Matrix shared by the slices of a batch operation must be a leaf (weight or input)");
    }
  }
  if (D > 1 && op == PRAD_OP_MATMUL)
    PRAD_REQUIRE(a.depth == D || V[in_values[1]].depth == D, PRAD_ERR_SHAPE, "prad_graph_add_node: no operand has the output's depth");
  if (D > 1 && op != PRAD_OP_MATMUL)
    PRAD_REQUIRE(a.depth == D, PRAD_ERR_SHAPE, "prad_graph_add_node: the first input has to carry the slices");
  // shape rules of the managed operations
  bool ok = true;
  switch (op) {
    case PRAD_OP_MATMUL: {
      const GValue& b = V[in_values[1]];
      PRAD_REQUIRE(a.cols == b.rows, PRAD_ERR_SHAPE, "Input 1 columns do not match Input 2 rows");
      ok = o.rows == a.rows && o.cols == b.cols;
      break;
    }
    case PRAD_OP_ADD_BROADCAST: {
      const GValue& b = V[in_values[1]];
      PRAD_REQUIRE(b.rows == 1 && b.cols == a.cols, PRAD_ERR_SHAPE,
                   "The length of the bias vector must be the same as the number of columns in the input matrix.");
      ok = o.rows == a.rows && o.cols == a.cols;
      break;
    }
    case PRAD_OP_TRANSPOSE: ok = o.rows == a.cols && o.cols == a.rows; break;
    default:
      for (int i = 1; i < n_in; ++i) ok = ok && V[in_values[i]].rows == a.rows && V[in_values[i]].cols == a.cols;
      ok = ok && o.rows == a.rows && o.cols == a.cols;
  }
  PRAD_REQUIRE(ok, PRAD_ERR_SHAPE, "prad_graph_add_node: operand shapes do not fit operation %d", (int)op);
  if (!o.data) {
    prad_status s = g_alloc(g, (size_t)o.count(), &o.data);
    if (s) return s;
    o.owned = true;
  }
  GNode n;
  n.op = op;
  n.in.assign(in_values, in_values + n_in);
  n.out = out_value;
  n.scalar = scalar;
  n.in_grad.assign(n_in, nullptr);
  g->nodes.push_back(n);
  g->values[out_value].produced_by = (int)g->nodes.size() - 1;
  if (out_node) *out_node = (int)g->nodes.size() - 1;
  return PRAD_OK;
}

prad_status prad_graph_value_data(prad_graph* g, int value, void** out_data) {
  PRAD_CHECK_GRAPH(g);
  PRAD_REQUIRE(value >= 0 && value < (int)g->values.size() && out_data, PRAD_ERR_INVALID, "prad_graph_value_data: bad argument");
  *out_data = g->values[value].data;
  return PRAD_OK;
}

prad_status prad_graph_value_gradient(prad_graph* g, int value, void** out_grad) {
  PRAD_CHECK_GRAPH(g);
  PRAD_REQUIRE(value >= 0 && value < (int)g->values.size() && out_grad, PRAD_ERR_INVALID, "prad_graph_value_gradient: bad argument");
  *out_grad = g->values[value].grad;
  return PRAD_OK;
}

prad_status prad_graph_consumer_count(prad_graph* g, int value, int* out_count) {
  PRAD_CHECK_GRAPH(g);
  PRAD_REQUIRE(value >= 0 && value < (int)g->values.size() && out_count, PRAD_ERR_INVALID, "prad_graph_consumer_count: bad argument");
  *out_count = g->values[value].consumers;
  return PRAD_OK;
}

}  // extern "C"

// ---------------------------------------------------------------- forward / backward walks
namespace prad {

#define G_TRY(call)                   \
  do {                                \
    prad_status s_ = (call);          \
    if (s_ != PRAD_OK) return s_;     \
  } while (0)

static prad_status node_forward(prad_graph* g, GNode& n) {
  auto& V = g->values;
  prad_ctx* c = g->ctx;
  const prad_dtype dt = g->dt;
  GValue& o = V[n.out];
  const GValue& a = V[n.in[0]];
  const int64_t cnt = o.count();
  const int D = o.depth;
  const int64_t rows_all = (int64_t)D * a.rows;      // rows of all slices for the row-wise operations
  switch (n.op) {
    case PRAD_OP_MATMUL: {
      const GValue& b = V[n.in[1]];
      if (D == 1)
        return prad_matmul_forward(c, dt, a.data, b.data, o.data, a.rows, a.cols, b.cols, nullptr, nullptr, PRAD_ACT_NONE, 0.0);
      if (a.depth == D)    // (DeepMatrix, DeepMatrix) and (DeepMatrix, Matrix)
        return prad_batch_matmul_forward(c, dt, a.data, b.data, o.data, D, a.rows, a.cols, b.cols, b.depth == 1);
      // (Matrix, DeepMatrix): every slice is multiplied from the left by the same matrix
      return prad_gemm(c, dt, 0, 0, a.rows, b.cols, a.cols, 1.0, a.data, a.cols, b.data, b.cols, 0.0, o.data, b.cols, D, 0,
                       b.slice(), o.slice());
    }
    case PRAD_OP_ADD:
      if (V[n.in[1]].depth != D)   // (DeepMatrix, Matrix): the matrix is a "row" added to each of the D slices
        return prad_add_broadcast_forward(c, dt, a.data, V[n.in[1]].data, o.data, D, (int)a.slice());
      return prad_add_forward(c, dt, a.data, V[n.in[1]].data, nullptr, o.data, cnt);
    case PRAD_OP_ADD3:
      if (V[n.in[2]].depth != D) {   // (a + b) + bias, the bias shared by the slices
        G_TRY(prad_add_forward(c, dt, a.data, V[n.in[1]].data, nullptr, o.data, cnt));
        return prad_add_broadcast_forward(c, dt, o.data, V[n.in[2]].data, o.data, D, (int)a.slice());
      }
      return prad_add_forward(c, dt, a.data, V[n.in[1]].data, V[n.in[2]].data, o.data, cnt);
    case PRAD_OP_ADD_BROADCAST:
      return prad_add_broadcast_forward(c, dt, a.data, V[n.in[1]].data, o.data, (int)rows_all, a.cols);
    case PRAD_OP_HADAMARD: return prad_hadamard_forward(c, dt, a.data, V[n.in[1]].data, o.data, cnt);
    case PRAD_OP_LEAKY_RELU: case PRAD_OP_SIGMOID: case PRAD_OP_TANH: case PRAD_OP_GELU:
    case PRAD_OP_RELU: case PRAD_OP_AMPLIFIED_SIGMOID:
      return prad_act_forward(c, dt, act_of(n.op), a.data, o.data, cnt, n.scalar);
    case PRAD_OP_SOFTMAX: return prad_softmax_forward(c, dt, a.data, o.data, rows_all, a.cols);
    case PRAD_OP_SINE_SOFTMAX: return prad_sine_softmax_forward(c, dt, a.data, o.data, rows_all, a.cols);
    case PRAD_OP_LAYERNORM:
      if (!n.aux0) {
        G_TRY(g_alloc(g, (size_t)rows_all, &n.aux0));
        G_TRY(g_alloc(g, (size_t)rows_all, &n.aux1));
      }
      return prad_layernorm_forward(c, dt, a.data, o.data, n.aux0, n.aux1, rows_all, a.cols);
    case PRAD_OP_SCALE: return prad_scale(c, dt, a.data, o.data, cnt, n.scalar);
    case PRAD_OP_TRANSPOSE: return prad_transpose(c, dt, a.data, o.data, a.rows, a.cols, D);
  }
  return PRAD_ERR_INVALID;
}

// gradient buffer of input i of node n (allocated once)
static prad_status in_grad_buf(prad_graph* g, GNode& n, int i, void** out) {
  if (!n.in_grad[i]) {
    const GValue& v = g->values[n.in[i]];
    G_TRY(g_alloc(g, (size_t)v.count(), &n.in_grad[i]));
  }
  *out = n.in_grad[i];
  return PRAD_OK;
}

// Runs the Backward of one node for upstream gradient d (shape of its output) and hands each
// input's gradient to that input value.  MatrixAdd-style operations pass d on by reference,
// exactly as MatrixAddBroadcastingOperation.Backward returns dOutput itself.
// mean over the D slices of `deep` (D x per elements) into `out` (per elements): the visitor's combined
// gradient of a Matrix shared by the slices of a batch operation (sum of the slices times 1/D)
static prad_status slice_mean(prad_graph* g, const void* deep, void* out, int D, int64_t per) {
  G_TRY(prad_add_broadcast_backward(g->ctx, g->dt, deep, out, D, (int)per, 0));
  return prad_scale(g->ctx, g->dt, out, out, per, 1.0 / (double)D);
}

static prad_status node_backward(prad_graph* g, GNode& n, void* d) {
  auto& V = g->values;
  prad_ctx* c = g->ctx;
  const prad_dtype dt = g->dt;
  const GValue& o = V[n.out];
  const GValue& a = V[n.in[0]];
  const int64_t cnt = o.count();
  const int D = o.depth;
  const int64_t rows_all = (int64_t)D * a.rows;
  void* ga = nullptr;
  void* gb = nullptr;
  switch (n.op) {
    case PRAD_OP_MATMUL: {
      const GValue& b = V[n.in[1]];
      G_TRY(in_grad_buf(g, n, 0, &ga));
      G_TRY(in_grad_buf(g, n, 1, &gb));
      const int M = a.rows, K = a.cols, N = b.cols;
      if (D == 1) {
        G_TRY(prad_matmul_backward(c, dt, a.data, b.data, d, ga, gb, M, K, N, 0, 1.0, PRAD_ACT_NONE, nullptr, 0.0));
      } else if (a.depth == D && b.depth == D) {
        G_TRY(prad_batch_matmul_backward(c, dt, a.data, b.data, d, ga, gb, nullptr, D, M, K, N, 0));
      } else if (a.depth == D) {   // shared second operand: its gradient is the mean of the slices' A_d^T dC_d
        G_TRY(prad_batch_matmul_backward(c, dt, a.data, b.data, d, ga, nullptr, gb, D, M, K, N, 1));
      } else {                     // shared first operand W: dX_d = W^T dC_d ; dW = (1/D) sum_d dC_d X_d^T
        G_TRY(prad_gemm(c, dt, 1, 0, K, N, M, 1.0, a.data, K, d, N, 0.0, gb, N, D, 0, o.slice(), b.slice()));
        if (N == 1) {              // column vectors: the slices of dC and X are the rows of two matrices
          G_TRY(prad_gemm(c, dt, 1, 0, M, K, D, 1.0 / (double)D, d, M, b.data, K, 0.0, ga, K, 1, 0, 0, 0));
        } else {
          if (!n.aux0) G_TRY(g_alloc(g, (size_t)D * M * K, &n.aux0));
          G_TRY(prad_gemm(c, dt, 0, 1, M, K, N, 1.0, d, N, b.data, N, 0.0, n.aux0, K, D, o.slice(), b.slice(), (int64_t)M * K));
          G_TRY(slice_mean(g, n.aux0, ga, D, (int64_t)M * K));
        }
      }
      V[n.in[0]].contrib.push_back(ga);
      V[n.in[1]].contrib.push_back(gb);
      return PRAD_OK;
    }
    case PRAD_OP_ADD: case PRAD_OP_ADD3:
      for (size_t i = 0; i < n.in.size(); ++i) {
        GValue& iv = V[n.in[i]];
        if (iv.depth == D) {
          iv.contrib.push_back(d);
        } else {                   // the Matrix shared by the slices
          void* gs = nullptr;
          G_TRY(in_grad_buf(g, n, (int)i, &gs));
          G_TRY(slice_mean(g, d, gs, D, iv.slice()));
          iv.contrib.push_back(gs);
        }
      }
      return PRAD_OK;
    case PRAD_OP_ADD_BROADCAST:
      G_TRY(in_grad_buf(g, n, 1, &gb));
      G_TRY(prad_add_broadcast_backward(c, dt, d, gb, (int)rows_all, o.cols, 0));
      if (D > 1) G_TRY(prad_scale(c, dt, gb, gb, o.cols, 1.0 / (double)D));   // mean of the slices' column sums
      V[n.in[0]].contrib.push_back(d);
      V[n.in[1]].contrib.push_back(gb);
      return PRAD_OK;
    case PRAD_OP_HADAMARD:
      G_TRY(in_grad_buf(g, n, 0, &ga));
      G_TRY(in_grad_buf(g, n, 1, &gb));
      G_TRY(prad_hadamard_backward(c, dt, a.data, V[n.in[1]].data, d, ga, gb, cnt));
      V[n.in[0]].contrib.push_back(ga);
      V[n.in[1]].contrib.push_back(gb);
      return PRAD_OK;
    case PRAD_OP_LEAKY_RELU: case PRAD_OP_GELU: case PRAD_OP_RELU: case PRAD_OP_AMPLIFIED_SIGMOID:   // Backward reads the input
      G_TRY(in_grad_buf(g, n, 0, &ga));
      G_TRY(prad_act_backward(c, dt, act_of(n.op), a.data, d, ga, cnt, n.scalar));
      break;
    case PRAD_OP_SIGMOID: case PRAD_OP_TANH:        // Backward reads the output
      G_TRY(in_grad_buf(g, n, 0, &ga));
      G_TRY(prad_act_backward(c, dt, act_of(n.op), o.data, d, ga, cnt, n.scalar));
      break;
    case PRAD_OP_SOFTMAX:
      G_TRY(in_grad_buf(g, n, 0, &ga));
      G_TRY(prad_softmax_backward(c, dt, o.data, d, ga, rows_all, o.cols));
      break;
    case PRAD_OP_SINE_SOFTMAX:                      // Backward reads the input
      G_TRY(in_grad_buf(g, n, 0, &ga));
      G_TRY(prad_sine_softmax_backward(c, dt, a.data, d, ga, rows_all, o.cols));
      break;
    case PRAD_OP_LAYERNORM:
      PRAD_REQUIRE(n.aux0, PRAD_ERR_INVALID, "prad_graph_backward: LayerNorm node has no forward state (run prad_graph_forward)");
      G_TRY(in_grad_buf(g, n, 0, &ga));
      G_TRY(prad_layernorm_backward(c, dt, a.data, n.aux0, n.aux1, d, ga, rows_all, a.cols));
      break;
    case PRAD_OP_SCALE:
      G_TRY(in_grad_buf(g, n, 0, &ga));
      G_TRY(prad_scale(c, dt, d, ga, cnt, n.scalar));
      break;
    case PRAD_OP_TRANSPOSE:
      G_TRY(in_grad_buf(g, n, 0, &ga));
      G_TRY(prad_transpose(c, dt, d, ga, o.rows, o.cols, D));
      break;
  }
  V[n.in[0]].contrib.push_back(ga);
  return PRAD_OK;
}

}  // namespace prad

extern "C" {

prad_status prad_graph_forward(prad_graph* g) {
  PRAD_CHECK_GRAPH(g);
  for (GNode& n : g->nodes) {
    for (int i : n.in)
      PRAD_REQUIRE(g->values[i].data, PRAD_ERR_INVALID, "prad_graph_forward: value %d has no data and no producer before its use", i);
    G_TRY(node_forward(g, n));
  }
  return PRAD_OK;
}

prad_status prad_graph_backward_multi(prad_graph* g, const int* start_values, const void* const* d_starts, int count) {
  PRAD_CHECK_GRAPH(g);
  auto& V = g->values;
  PRAD_REQUIRE(count >= 1 && start_values && d_starts, PRAD_ERR_INVALID, "prad_graph_backward: no start value");
  for (int i = 0; i < count; ++i) {
    PRAD_REQUIRE(start_values[i] >= 0 && start_values[i] < (int)V.size() && d_starts[i], PRAD_ERR_INVALID,
                 "prad_graph_backward: bad start value or null gradient at position %d", i);
    for (int j = 0; j < i; ++j)
      PRAD_REQUIRE(start_values[j] != start_values[i], PRAD_ERR_INVALID, "prad_graph_backward: start value %d is listed twice",
                   start_values[i]);
  }
  // 1. which nodes lie on a path to a start value, and how many consumers each value has
  //    there (OperationGraphVisitor's dependency counts)
  std::vector<char> needed(V.size(), 0), is_start(V.size(), 0);
  for (int i = 0; i < count; ++i) needed[start_values[i]] = is_start[start_values[i]] = 1;
  for (GValue& v : V) { v.contrib.clear(); v.grad = nullptr; v.consumers = 0; }
  std::vector<char> live(g->nodes.size(), 0);
  for (int k = (int)g->nodes.size() - 1; k >= 0; --k) {
    GNode& n = g->nodes[k];
    if (!needed[n.out]) continue;
    live[k] = 1;
    for (int i : n.in) { needed[i] = 1; V[i].consumers++; }
  }
  // 2. one reverse walk.  Nodes were added in forward order, so every consumer of a value
  //    has delivered its contribution before the value's producer is reached; contributions
  //    arrive in reverse consumer order and are summed in consumer (registration) order, an
  //    upstream gradient handed in by the caller first.
  auto finalize = [&](GValue& v, const void* external) -> prad_status {
    if (v.contrib.empty() && !external) return PRAD_OK;
    std::reverse(v.contrib.begin(), v.contrib.end());
    if (external) v.contrib.insert(v.contrib.begin(), const_cast<void*>(external));
    if (v.contrib.size() == 1) {
      v.grad = v.contrib[0];
    } else {
      if (!v.sum_buf) G_TRY(g_alloc(g, (size_t)v.count(), &v.sum_buf));
      G_TRY(prad_segmented_sum(g->ctx, g->dt, v.contrib.data(), (int)v.contrib.size(), v.sum_buf, v.count()));
      v.grad = v.sum_buf;
    }
    if (v.grad_dst) G_TRY(prad_accumulate(g->ctx, g->dt, v.grad_dst, v.grad, v.count()));
    return PRAD_OK;
  };
  auto external_of = [&](int value) -> const void* {
    if (!is_start[value]) return nullptr;
    for (int i = 0; i < count; ++i)
      if (start_values[i] == value) return d_starts[i];
    return nullptr;
  };
  for (int k = (int)g->nodes.size() - 1; k >= 0; --k) {
    if (!live[k]) continue;
    GNode& n = g->nodes[k];
    GValue& o = V[n.out];
    G_TRY(finalize(o, external_of(n.out)));
    PRAD_REQUIRE(o.grad, PRAD_ERR_INVALID, "prad_graph_backward: node %d is on the path but received no gradient", k);
    G_TRY(node_backward(g, n, o.grad));
  }
  // 3. leaves (inputs, weights): fan-in sum and `destination += gradient`
  for (size_t i = 0; i < V.size(); ++i)
    if (V[i].produced_by < 0 && (needed[i] || is_start[i])) G_TRY(finalize(V[i], external_of((int)i)));
  return PRAD_OK;
}

prad_status prad_graph_backward(prad_graph* g, int start_value, const void* d_start) {
  return prad_graph_backward_multi(g, &start_value, &d_start, 1);
}

}  // extern "C"
