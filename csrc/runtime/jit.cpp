// JIT expression trees: build, symbolic derivative, text (de)serialisation, CPU interpreter and CUDA C++
// code generation for one fused element-wise kernel.
//
// Same 18 node kinds and the same text format as the reference (include/litetorch/jit.h:13-178,
// src/ops/jit.cpp:601-670): a tree is written in prefix order as "op name val left right" with "N" for a
// missing child and "_" for an empty name; the older parenthesised form "(op,name,val,left,right)" found in
// saved files is read as well.  The reference generates a fused kernel for OpenCL only and evaluates node by
// node on CUDA (src/ops/jit.cpp:279-327); here `lt_jit_cuda_source` emits one CUDA kernel for the whole tree,
// which the CUDA-side runtime compiles with NVRTC and caches.
#include "lt_host.h"

#include <cmath>
#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <sstream>
#include <string>
#include <vector>

namespace {

enum Op : int {
  INPUT = 0, CONST = 1, ADD = 2, SUB = 3, MUL = 4, DIV = 5, RELU = 6, GELU = 7, SIGMOID = 8, TANH = 9, SQRT = 10,
  EXP = 11, LOG = 12, ABS = 13, NEG = 14, RELU_GRAD = 15, GELU_GRAD = 16, ABS_GRAD = 17
};

struct Node {
  int op;
  std::string name;
  float val = 0.f;
  int left = -1, right = -1;
};

std::vector<Node> g_nodes;
std::mutex g_mu;

int make(int op, const std::string& name, float val, int l, int r) {
  g_nodes.push_back(Node{op, name, val, l, r});
  return int(g_nodes.size()) - 1;
}
int cst(float v) { return make(CONST, "", v, -1, -1); }
int bin(int op, int a, int b) { return make(op, "", 0.f, a, b); }
int un(int op, int a) { return make(op, "", 0.f, a, -1); }

bool is_const(int n, float v) { return n >= 0 && g_nodes[n].op == CONST && g_nodes[n].val == v; }

// light algebraic clean-up so that derivatives stay readable
int s_add(int a, int b) { if (is_const(a, 0.f)) return b; if (is_const(b, 0.f)) return a; return bin(ADD, a, b); }
int s_sub(int a, int b) { if (is_const(b, 0.f)) return a; if (is_const(a, 0.f)) return un(NEG, b); return bin(SUB, a, b); }
int s_mul(int a, int b) {
  if (is_const(a, 0.f) || is_const(b, 0.f)) return cst(0.f);
  if (is_const(a, 1.f)) return b;
  if (is_const(b, 1.f)) return a;
  return bin(MUL, a, b);
}
int s_div(int a, int b) { if (is_const(a, 0.f)) return cst(0.f); if (is_const(b, 1.f)) return a; return bin(DIV, a, b); }

int derive(int n, const std::string& wrt) {
  if (n < 0) return cst(0.f);
  const Node nd = g_nodes[n];
  const int u = nd.left, v = nd.right;
  switch (nd.op) {
    case INPUT: return cst(nd.name == wrt ? 1.f : 0.f);
    case CONST: return cst(0.f);
    case ADD: return s_add(derive(u, wrt), derive(v, wrt));
    case SUB: return s_sub(derive(u, wrt), derive(v, wrt));
    case MUL: return s_add(s_mul(derive(u, wrt), v), s_mul(u, derive(v, wrt)));
    case DIV: return s_div(s_sub(s_mul(derive(u, wrt), v), s_mul(u, derive(v, wrt))), s_mul(v, v));
    case RELU: return s_mul(un(RELU_GRAD, u), derive(u, wrt));
    case GELU: return s_mul(un(GELU_GRAD, u), derive(u, wrt));
    case SIGMOID: { int s = un(SIGMOID, u); return s_mul(s_mul(s, s_sub(cst(1.f), s)), derive(u, wrt)); }
    case TANH: { int t = un(TANH, u); return s_mul(s_sub(cst(1.f), s_mul(t, t)), derive(u, wrt)); }
    case SQRT: return s_div(derive(u, wrt), s_mul(cst(2.f), un(SQRT, u)));
    case EXP: return s_mul(un(EXP, u), derive(u, wrt));
    case LOG: return s_div(derive(u, wrt), u);
    case ABS: return s_mul(un(ABS_GRAD, u), derive(u, wrt));
    case NEG: return un(NEG, derive(u, wrt));
    default: return cst(0.f);  // the *_GRAD helper nodes are piecewise constant / not differentiated further
  }
}

float gelu_f(float x) { const float k0 = 0.7978845608028654f, k1 = 0.044715f; return 0.5f * x * (1.f + std::tanh(k0 * (x + k1 * x * x * x))); }
float gelu_grad_f(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float t = std::tanh(k0 * (x + k1 * x * x * x));
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * k0 * (1.f + 3.f * k1 * x * x);
}

float eval(int n, const std::map<std::string, const float*>& env, uint64_t i) {
  const Node& nd = g_nodes[n];
  switch (nd.op) {
    case INPUT: { auto it = env.find(nd.name); return it == env.end() ? 0.f : it->second[i]; }
    case CONST: return nd.val;
    case ADD: return eval(nd.left, env, i) + eval(nd.right, env, i);
    case SUB: return eval(nd.left, env, i) - eval(nd.right, env, i);
    case MUL: return eval(nd.left, env, i) * eval(nd.right, env, i);
    case DIV: return eval(nd.left, env, i) / eval(nd.right, env, i);
    case RELU: { float x = eval(nd.left, env, i); return x > 0.f ? x : 0.f; }
    case GELU: return gelu_f(eval(nd.left, env, i));
    case SIGMOID: return 1.f / (1.f + std::exp(-eval(nd.left, env, i)));
    case TANH: return std::tanh(eval(nd.left, env, i));
    case SQRT: return std::sqrt(eval(nd.left, env, i));
    case EXP: return std::exp(eval(nd.left, env, i));
    case LOG: return std::log(eval(nd.left, env, i));
    case ABS: return std::fabs(eval(nd.left, env, i));
    case NEG: return -eval(nd.left, env, i);
    case RELU_GRAD: return eval(nd.left, env, i) > 0.f ? 1.f : 0.f;
    case GELU_GRAD: return gelu_grad_f(eval(nd.left, env, i));
    case ABS_GRAD: { float x = eval(nd.left, env, i); return x > 0.f ? 1.f : (x < 0.f ? -1.f : 0.f); }
  }
  return 0.f;
}

void serialize(int n, std::ostringstream& os) {
  if (n < 0) { os << "N"; return; }
  const Node& nd = g_nodes[n];
  os << nd.op << " " << (nd.name.empty() ? "_" : nd.name) << " " << nd.val << " ";
  serialize(nd.left, os);
  os << " ";
  serialize(nd.right, os);
}

int parse_spaces(std::istringstream& is) {
  std::string tok;
  if (!(is >> tok) || tok == "N") return -1;
  const int op = std::stoi(tok);
  std::string name;
  is >> name;
  if (name == "_") name.clear();
  float val = 0.f;
  is >> val;
  const int l = parse_spaces(is);
  const int r = parse_spaces(is);
  return make(op, name, val, l, r);
}

// "(op,name,val,left,right)" or "N"
int parse_paren(const std::string& s, size_t& pos) {
  while (pos < s.size() && isspace(static_cast<unsigned char>(s[pos]))) ++pos;
  if (pos < s.size() && s[pos] == 'N') { ++pos; return -1; }
  if (pos >= s.size() || s[pos] != '(') return -1;
  ++pos;
  auto field = [&]() { size_t e = s.find(',', pos); std::string f = s.substr(pos, e - pos); pos = e + 1; return f; };
  const int op = std::stoi(field());
  const std::string name = field();
  const float val = std::stof(field());
  const int l = parse_paren(s, pos);
  if (pos < s.size() && s[pos] == ',') ++pos;
  const int r = parse_paren(s, pos);
  if (pos < s.size() && s[pos] == ')') ++pos;
  return make(op, name, val, l, r);
}

void emit(int n, std::ostringstream& os) {
  if (n < 0) { os << "0.0f"; return; }
  const Node& nd = g_nodes[n];
  auto un_fn = [&](const char* fn) { os << fn << "("; emit(nd.left, os); os << ")"; };
  auto bin_op = [&](const char* op) { os << "("; emit(nd.left, os); os << " " << op << " "; emit(nd.right, os); os << ")"; };
  switch (nd.op) {
    case INPUT: os << "v_" << nd.name; break;
    case CONST: { std::ostringstream t; t.precision(9); t << std::scientific << nd.val; os << t.str() << "f"; break; }
    case ADD: bin_op("+"); break;
    case SUB: bin_op("-"); break;
    case MUL: bin_op("*"); break;
    case DIV: bin_op("/"); break;
    case RELU: un_fn("lt_relu"); break;
    case GELU: un_fn("lt_gelu"); break;
    case SIGMOID: un_fn("lt_sigmoid"); break;
    case TANH: un_fn("tanhf"); break;
    case SQRT: un_fn("sqrtf"); break;
    case EXP: un_fn("__expf"); break;
    case LOG: un_fn("__logf"); break;
    case ABS: un_fn("fabsf"); break;
    case NEG: os << "(-"; emit(nd.left, os); os << ")"; break;
    case RELU_GRAD: un_fn("lt_relu_grad"); break;
    case GELU_GRAD: un_fn("lt_gelu_grad"); break;
    case ABS_GRAD: un_fn("lt_sign"); break;
  }
}

int copy_out(const std::string& s, char* buf, int cap) {
  if (int(s.size()) + 1 > cap) return -int(s.size()) - 1;
  memcpy(buf, s.c_str(), s.size() + 1);
  return int(s.size());
}

}  // namespace

extern "C" {

int lt_jit_input(const char* name) { std::lock_guard<std::mutex> lk(g_mu); return make(INPUT, name, 0.f, -1, -1); }
int lt_jit_const(float v) { std::lock_guard<std::mutex> lk(g_mu); return cst(v); }
int lt_jit_binary(int op, int a, int b) { std::lock_guard<std::mutex> lk(g_mu); return bin(op, a, b); }
int lt_jit_unary(int op, int a) { std::lock_guard<std::mutex> lk(g_mu); return un(op, a); }
int lt_jit_derivative(int node, const char* wrt) { std::lock_guard<std::mutex> lk(g_mu); return derive(node, wrt); }
int lt_jit_node_op(int node) { std::lock_guard<std::mutex> lk(g_mu); return node >= 0 && node < int(g_nodes.size()) ? g_nodes[node].op : -1; }
float lt_jit_node_val(int node) { std::lock_guard<std::mutex> lk(g_mu); return node >= 0 && node < int(g_nodes.size()) ? g_nodes[node].val : 0.f; }
int lt_jit_node_left(int node) { std::lock_guard<std::mutex> lk(g_mu); return node >= 0 && node < int(g_nodes.size()) ? g_nodes[node].left : -1; }
int lt_jit_node_right(int node) { std::lock_guard<std::mutex> lk(g_mu); return node >= 0 && node < int(g_nodes.size()) ? g_nodes[node].right : -1; }
int lt_jit_node_name(int node, char* buf, int cap) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (node < 0 || node >= int(g_nodes.size())) return -1;
  return copy_out(g_nodes[node].name, buf, cap);
}

// Returns the length written, or -(needed) when the buffer is too small.
int lt_jit_serialize(int node, char* buf, int cap) {
  std::lock_guard<std::mutex> lk(g_mu);
  std::ostringstream os;
  serialize(node, os);
  return copy_out(os.str(), buf, cap);
}
int lt_jit_deserialize(const char* text) {
  std::lock_guard<std::mutex> lk(g_mu);
  std::string s(text);
  size_t first = s.find_first_not_of(" \t\r\n");
  if (first == std::string::npos) return -1;
  try {
    if (s[first] == '(') { size_t pos = first; return parse_paren(s, pos); }
    std::istringstream is(s);
    return parse_spaces(is);
  } catch (...) {
    return -1;
  }
}

// out[i] = tree(inputs[*][i]) for i < n; names/ptrs describe the inputs.
int lt_jit_eval_cpu(int node, const char* const* names, const float* const* ptrs, int n_inputs, uint64_t n, float* out) {
  std::map<std::string, const float*> env;
  for (int i = 0; i < n_inputs; ++i) env[names[i]] = ptrs[i];
  std::lock_guard<std::mutex> lk(g_mu);
  for (uint64_t i = 0; i < n; ++i) out[i] = eval(node, env, i);
  return 0;
}

// CUDA C++ source of `extern "C" __global__ void <kernel>(const T* in0, ..., T* out, long long n)` where T is
// float (dtype 0) or __nv_bfloat16 (dtype 1); math is fp32 either way.  Inputs appear in the order of `names`.
int lt_jit_cuda_source(int node, const char* const* names, int n_inputs, const char* kernel, int dtype, char* buf, int cap) {
  std::lock_guard<std::mutex> lk(g_mu);
  std::ostringstream os;
  os << "#include <cuda_bf16.h>\n"
        "__device__ __forceinline__ float lt_relu(float x) { return x > 0.f ? x : 0.f; }\n"
        "__device__ __forceinline__ float lt_relu_grad(float x) { return x > 0.f ? 1.f : 0.f; }\n"
        "__device__ __forceinline__ float lt_sign(float x) { return x > 0.f ? 1.f : (x < 0.f ? -1.f : 0.f); }\n"
        "__device__ __forceinline__ float lt_sigmoid(float x) { return 1.f / (1.f + __expf(-x)); }\n"
        "__device__ __forceinline__ float lt_gelu(float x) { const float k0 = 0.7978845608028654f, k1 = 0.044715f;"
        " return 0.5f * x * (1.f + tanhf(k0 * (x + k1 * x * x * x))); }\n"
        "__device__ __forceinline__ float lt_gelu_grad(float x) { const float k0 = 0.7978845608028654f, k1 = 0.044715f;"
        " const float t = tanhf(k0 * (x + k1 * x * x * x));"
        " return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * k0 * (1.f + 3.f * k1 * x * x); }\n";
  const char* T = dtype == 1 ? "__nv_bfloat16" : "float";
  os << "extern \"C\" __global__ void " << kernel << "(";
  for (int i = 0; i < n_inputs; ++i) os << "const " << T << "* __restrict__ in" << i << ", ";
  os << T << "* __restrict__ out, long long n) {\n"
     << "  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {\n";
  for (int i = 0; i < n_inputs; ++i) {
    os << "    const float v_" << names[i] << " = ";
    if (dtype == 1) os << "__bfloat162float(in" << i << "[i]);\n"; else os << "in" << i << "[i];\n";
  }
  os << "    const float r = ";
  emit(node, os);
  os << ";\n";
  if (dtype == 1) os << "    out[i] = __float2bfloat16(r);\n"; else os << "    out[i] = r;\n";
  os << "  }\n}\n";
  return copy_out(os.str(), buf, cap);
}

}  // extern "C"
