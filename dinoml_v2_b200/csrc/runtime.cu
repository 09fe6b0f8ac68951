// Artifact / session runtime: the `dino_*` C ABI over an interpreted launch plan.
//
// The reference generates one module.so per model from src/dinoml/templates/gpu_module.cu.j2 (module
// and session structs, constant loading, per-run validation, the launch sequence, a CUDA-graph
// benchmark loop).  This runtime provides the same entry points from one prebuilt library: the
// artifact directory carries `module_plan.txt`, a line-based description of tensors, constants and
// gemm nodes written by the Python compiler, and a session walks it - one fused launch per
// quantized linear on the session stream, no dequantization scratch.
//
// Plan grammar (whitespace-separated tokens, one record per line):
//   dinoml_b200_module_plan 1
//   tensor <name> input|output|temp <DinoDtype> <ndim> <dim>...          dim = N  or  ?min:max
//   constant <name> dense <DinoDtype> <offset> <nbytes> <ndim> <dim>...
//   constant <name> gguf <qtype_value> <offset> <nbytes> <rows> <n_per_row> <residency>
//   node gemm_rcr <a> <b> <bias|-> <out> <variant>                       also gemm_rcr_bias; dual_gemm_rcr_silu / _fast_gelu with
//                                                                         <b> = the two weights' rows interleaved in groups of 8
//   dispatch <node_index> <m> <n> <k> <variant>                          shape-guarded selection
//
// Where an encoded constant lives (its <residency>; policy names of src/dinoml/constant_sources.py:17-34, which the
// reference declares but does not implement):
//   manual_runtime_load / eager_encoded_device   on the device from load time on;
//   cpu_until_first_use    in pinned host memory until the first run that needs it, then on the device for good;
//   sequential_offload     in pinned host memory; a run streams each weight into one of two device slots just ahead of
//                          its launch (the next weight is copied on a second stream while the current one computes);
//   grouped_offload        the same at the granularity of groups of constants (one group = e.g. one layer).
// Steady state: dino_session_set_graph_replay(session, 1) makes dino_session_run capture the launch sequence of a
// (shapes, pointers) combination the second time it sees it and replay the graph from then on.
// DINOML_PROFILE_RUN[_VERBOSE|_SECTIONS] time every launch with events, as src/dinoml/templates/gpu_module.cu.j2:785-983.
#if defined(__SSE2__)
#include <emmintrin.h>
#endif
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <sstream>
#include <string>
#include <vector>

#include "../../include/dinoml_b200_runtime.h"
#include "gguf_common.cuh"

namespace b200gguf {
int set_error_message(int rc, const std::string& message);
const char* last_error();
int dual_gemm_rcr(const void* a, const void* b01, const void* bias01, void* c, int qtype, int dtype, int m, int n, int k, int activation,
                  int variant, cudaStream_t s);
int gemm_rcr(const void* a, const void* b, const void* bias, void* c, int qtype, int dtype, int m, int n, int k,
             int variant, cudaStream_t s);
}  // namespace b200gguf

using b200gguf::set_error_message;

namespace {

int fail(const std::string& message) { return set_error_message(1, message); }
int cuda_fail(const char* what, cudaError_t err) { return fail(std::string(what) + ": " + cudaGetErrorString(err)); }

size_t dtype_size(int dtype) {
  switch (dtype) {
    case DINO_DTYPE_FLOAT16: case DINO_DTYPE_BFLOAT16: return 2;
    case DINO_DTYPE_FLOAT32: case DINO_DTYPE_INT32: return 4;
    case DINO_DTYPE_INT64: return 8;
    case DINO_DTYPE_BOOL: case DINO_DTYPE_FLOAT8_E4M3: case DINO_DTYPE_FLOAT8_E5M2: return 1;
    default: return 0;
  }
}

struct DimSpec { int64_t min = 0, max = 0; bool dynamic() const { return min != max; } };

struct TensorSpec {
  std::string name;
  int role = 0;  // 0 input, 1 output, 2 temp
  int dtype = 0;
  std::vector<DimSpec> dims;
  size_t max_bytes() const {
    size_t n = dtype_size(dtype);
    for (const DimSpec& d : dims) n *= size_t(d.max);
    return n;
  }
};

struct ConstantSpec {
  std::string name;
  bool encoded = false;
  int dtype = 0;        // dense
  int qtype = 0;        // encoded
  size_t offset = 0, nbytes = 0;
  std::vector<int64_t> shape;   // dense: logical shape; encoded: {rows, n_per_row}
  std::string residency;
  void* device = nullptr;
  bool loaded = false;
  // host residency (cpu_until_first_use / sequential_offload / grouped_offload)
  int policy = 0;               // 0 device-resident, 1 first use, 2 offloaded through the module's two device slots
  void* host = nullptr;         // pinned copy of the encoded bytes, owned by the module
  int group = -1;               // offload group (policy 2)
  size_t slot_offset = 0;       // offset of this constant inside its group's slot image
};

enum : int { RES_DEVICE = 0, RES_FIRST_USE = 1, RES_OFFLOAD = 2 };
int residency_policy(const std::string& r) {
  if (r == "cpu_until_first_use") return RES_FIRST_USE;
  if (r == "sequential_offload" || r == "grouped_offload") return RES_OFFLOAD;
  return RES_DEVICE;
}

struct OffloadGroup { std::vector<int> constants; size_t bytes = 0; };
struct OffloadState {
  std::map<int, OffloadGroup> groups;         // by group id
  void* slot[2] = {nullptr, nullptr};
  size_t slot_bytes = 0;
  int resident[2] = {-1, -1};                 // group whose upload was last issued into each slot
  cudaStream_t copy_stream = nullptr;
  cudaEvent_t ready[2] = {nullptr, nullptr};  // recorded on the copy stream after an upload
  cudaEvent_t freed[2] = {nullptr, nullptr};  // recorded on a compute stream after the last launch that read the slot
  bool freed_valid[2] = {false, false};
  size_t uploads = 0, upload_bytes = 0, host_bytes = 0;
};

struct NodeSpec {
  int a = -1, out = -1;       // tensor indices
  int b = -1, bias = -1;      // constant indices
  int variant = 0;
  int activation = 0;         // 0: gemm_rcr[_bias]; 1 / 2: dual_gemm_rcr_silu / _fast_gelu on a row-interleaved weight
};
struct DispatchSpec { int node, m, n, k, variant; };

}  // namespace

struct DinoModule {
  std::string artifact_dir, metadata_json;
  std::vector<TensorSpec> tensors;
  std::vector<int> inputs, outputs;
  std::vector<ConstantSpec> constants;
  std::vector<NodeSpec> nodes;
  std::vector<DispatchSpec> dispatch;
  OffloadState offload;
  size_t generation = 0;        // bumped whenever constant buffers are released: captured graphs of older generations are dropped
};

struct DinoSession {
  DinoModule* module = nullptr;
  cudaStream_t owned_stream = nullptr, stream = nullptr;
  bool external_stream = false;
  std::vector<void*> temps;                         // per tensor index (temp role only)
  std::vector<std::vector<int64_t>> shapes;         // per tensor index, as of the last run
  std::vector<bool> output_shape_valid;
  // steady-state replay: one captured graph per (input shapes, input / output pointers) seen at least twice
  bool graph_replay = false;
  struct CachedGraph { cudaGraphExec_t exec = nullptr; int seen = 0; std::vector<std::vector<int64_t>> out_shapes; };
  std::map<std::vector<int64_t>, CachedGraph> graphs;
  size_t graph_launches = 0;
  size_t graph_generation = 0;
  std::vector<int64_t> pending_key;     // combination of the run in progress; counted as seen once that run has succeeded
};

namespace {

int find_tensor(const DinoModule& m, const std::string& name) {
  for (size_t i = 0; i < m.tensors.size(); ++i) if (m.tensors[i].name == name) return int(i);
  return -1;
}
int find_constant(const DinoModule& m, const std::string& name) {
  for (size_t i = 0; i < m.constants.size(); ++i) if (m.constants[i].name == name) return int(i);
  return -1;
}

bool parse_dim(const std::string& tok, DimSpec* out) {
  if (tok.empty()) return false;
  if (tok[0] == '?') {
    long long lo = 0, hi = 0;
    if (std::sscanf(tok.c_str(), "?%lld:%lld", &lo, &hi) != 2 || lo < 0 || hi < lo) return false;
    out->min = lo; out->max = hi;
    return true;
  }
  char* end = nullptr;
  const long long v = std::strtoll(tok.c_str(), &end, 10);
  if (*end != '\0' || v < 0) return false;
  out->min = out->max = v;
  return true;
}

int parse_plan(DinoModule* mod, const std::string& path) {
  std::ifstream in(path);
  if (!in) return fail("cannot open " + path);
  std::string line;
  bool header = false;
  int lineno = 0;
  while (std::getline(in, line)) {
    ++lineno;
    std::istringstream ls(line);
    std::string kind;
    if (!(ls >> kind) || kind[0] == '#') continue;
    const std::string where = path + ":" + std::to_string(lineno) + ": ";
    if (kind == "dinoml_b200_module_plan") {
      int version = 0;
      if (!(ls >> version) || version != 1) return fail(where + "unsupported plan version");
      header = true;
    } else if (kind == "tensor") {
      TensorSpec t;
      std::string role;
      size_t ndim = 0;
      if (!(ls >> t.name >> role >> t.dtype >> ndim)) return fail(where + "malformed tensor record");
      t.role = role == "input" ? 0 : role == "output" ? 1 : role == "temp" ? 2 : -1;
      if (t.role < 0 || dtype_size(t.dtype) == 0 || ndim == 0 || ndim > 8) return fail(where + "bad tensor role/dtype/rank");
      for (size_t i = 0; i < ndim; ++i) {
        std::string tok;
        DimSpec d;
        if (!(ls >> tok) || !parse_dim(tok, &d)) return fail(where + "bad tensor dimension");
        t.dims.push_back(d);
      }
      if (t.role == 0) mod->inputs.push_back(int(mod->tensors.size()));
      if (t.role == 1) mod->outputs.push_back(int(mod->tensors.size()));
      mod->tensors.push_back(t);
    } else if (kind == "constant") {
      ConstantSpec c;
      std::string storage;
      if (!(ls >> c.name >> storage)) return fail(where + "malformed constant record");
      if (storage == "dense") {
        size_t ndim = 0;
        if (!(ls >> c.dtype >> c.offset >> c.nbytes >> ndim) || dtype_size(c.dtype) == 0) return fail(where + "bad dense constant");
        size_t numel = 1;
        for (size_t i = 0; i < ndim; ++i) {
          long long d = 0;
          if (!(ls >> d) || d < 0) return fail(where + "bad constant dimension");
          c.shape.push_back(d);
          numel *= size_t(d);
        }
        if (numel * dtype_size(c.dtype) != c.nbytes) return fail(where + "dense constant byte size does not match its shape");
      } else if (storage == "gguf") {
        long long rows = 0, npr = 0;
        c.encoded = true;
        if (!(ls >> c.qtype >> c.offset >> c.nbytes >> rows >> npr >> c.residency)) return fail(where + "bad gguf constant");
        const int bs = b200gguf::qtype_block_size(c.qtype);
        if (bs == 0) return fail(where + "unsupported GGUF qtype " + std::to_string(c.qtype));
        if (rows <= 0 || npr <= 0 || npr % bs) return fail(where + "n_per_row is not a multiple of the block size");
        if (size_t(rows) * size_t(npr / bs) * size_t(b200gguf::qtype_block_bytes(c.qtype)) != c.nbytes)
          return fail(where + "encoded_nbytes does not match rows x n_per_row");
        c.shape = {rows, npr};
        static const char* const kResidencies[] = {"manual_runtime_load", "eager_encoded_device", "cpu_until_first_use", "sequential_offload",
                                                   "grouped_offload"};
        bool known = false;
        for (const char* r : kResidencies) known = known || c.residency == r;
        if (!known) return fail(where + "unknown residency " + c.residency);
        c.policy = residency_policy(c.residency);
      } else {
        return fail(where + "unknown constant storage " + storage);
      }
      mod->constants.push_back(c);
    } else if (kind == "node") {
      std::string op, a, b, bias, out;
      NodeSpec n;
      if (!(ls >> op >> a >> b >> bias >> out >> n.variant)) return fail(where + "malformed node record");
      if (op == "dual_gemm_rcr_silu" || op == "dual_gemm_rcr_bias_silu") n.activation = 1;
      else if (op == "dual_gemm_rcr_fast_gelu" || op == "dual_gemm_rcr_bias_fast_gelu") n.activation = 2;
      else if (op != "gemm_rcr" && op != "gemm_rcr_bias") return fail(where + "unsupported op " + op);
      if (n.activation != 0 && (bias != "-") != (op.find("_bias_") != std::string::npos))
        return fail(where + op + (bias == "-" ? " needs its interleaved bias constant" : " takes no bias"));
      n.a = find_tensor(*mod, a);
      n.out = find_tensor(*mod, out);
      n.b = find_constant(*mod, b);
      n.bias = bias == "-" ? -1 : find_constant(*mod, bias);
      if (n.a < 0 || n.out < 0 || n.b < 0 || (bias != "-" && n.bias < 0)) return fail(where + "node references an unknown tensor");
      if (!mod->constants[n.b].encoded) return fail(where + "gemm weight must be a GGUF-encoded constant");
      if (n.bias >= 0 && mod->constants[n.bias].encoded) return fail(where + "bias must be a dense constant");
      if (n.variant < 0 || (n.variant & 0xff) > 4 || n.variant > 0xffff) return fail(where + "bad variant");   // family | config << 8
      mod->nodes.push_back(n);
    } else if (kind == "dispatch") {
      DispatchSpec d;
      if (!(ls >> d.node >> d.m >> d.n >> d.k >> d.variant) || d.node < 0 || size_t(d.node) >= mod->nodes.size() ||
          (d.variant & 0xff) < 1 || (d.variant & 0xff) > 4 || d.variant > 0xffff)
        return fail(where + "malformed dispatch record");
      mod->dispatch.push_back(d);
    } else {
      return fail(where + "unknown record " + kind);
    }
  }
  if (!header) return fail(path + ": missing plan header");
  if (mod->nodes.empty()) return fail(path + ": plan has no nodes");
  return 0;
}

int read_file(const std::string& path, std::string* out) {
  std::ifstream in(path, std::ios::binary);
  if (!in) return fail("cannot open " + path);
  std::ostringstream ss;
  ss << in.rdbuf();
  *out = ss.str();
  return 0;
}

int load_module(const char* artifact_dir, bool eager, DinoModule** out) {
  if (artifact_dir == nullptr || out == nullptr) return fail("dino_module_load received null pointer");
  *out = nullptr;
  DinoModule* mod = new DinoModule();
  mod->artifact_dir = artifact_dir;
  if (int rc = parse_plan(mod, mod->artifact_dir + "/module_plan.txt")) { delete mod; return rc; }
  if (int rc = read_file(mod->artifact_dir + "/metadata.json", &mod->metadata_json)) { delete mod; return rc; }
  if (eager) {
    if (int rc = dino_module_load_constants(mod, (mod->artifact_dir + "/constants.bin").c_str())) {
      dino_module_free(mod);
      return rc;
    }
  }
  *out = mod;
  return 0;
}

int ensure_constant_buffer(ConstantSpec& c) {
  if (c.device != nullptr || c.nbytes == 0) return 0;
  const cudaError_t err = cudaMalloc(&c.device, c.nbytes);
  return err == cudaSuccess ? 0 : cuda_fail("cudaMalloc (constant)", err);
}

int check_tensor(const TensorSpec& spec, const DinoTensor& t, const char* what, std::vector<int64_t>* shape) {
  const std::string who = std::string(what) + " '" + spec.name + "'";
  if (t.data == nullptr) return fail(who + " has a null data pointer");
  if (t.shape == nullptr) return fail(who + " has a null shape pointer");
  if (t.dtype != spec.dtype) return fail(who + " has dtype " + std::to_string(t.dtype) + ", expected " + std::to_string(spec.dtype));
  if (t.device_type != DINO_DEVICE_CUDA) return fail(who + " must live on a CUDA device");
  if (t.ndim != spec.dims.size()) return fail(who + " has rank " + std::to_string(t.ndim) + ", expected " + std::to_string(spec.dims.size()));
  shape->assign(t.shape, t.shape + t.ndim);
  size_t numel = 1;
  for (size_t i = 0; i < t.ndim; ++i) {
    if (t.shape[i] < spec.dims[i].min || t.shape[i] > spec.dims[i].max)
      return fail(who + " dimension " + std::to_string(i) + " = " + std::to_string(t.shape[i]) + " outside [" +
                  std::to_string(spec.dims[i].min) + ", " + std::to_string(spec.dims[i].max) + "]");
    numel *= size_t(t.shape[i]);
  }
  if (t.strides != nullptr) {  // contiguous row-major only, as runtime/include/dinoml/module_support.h:163-177
    int64_t expect = 1;
    for (size_t i = t.ndim; i-- > 0;) {
      if (t.shape[i] != 1 && t.strides[i] != expect) return fail(who + " must be contiguous");
      expect *= t.shape[i];
    }
  }
  const size_t esz = dtype_size(spec.dtype);
  if (t.byte_offset % esz) return fail(who + " byte_offset is not a multiple of the element size");
  if (t.nbytes != 0 && t.nbytes < numel * esz) return fail(who + " nbytes is smaller than its shape requires");
  return 0;
}

void* tensor_ptr(const DinoTensor& t) { return static_cast<uint8_t*>(t.data) + t.byte_offset; }

// ---- host-resident encoded constants -------------------------------------------------------------------------------
constexpr size_t kSlotAlign = 256;

// Lays the offload groups out (slot image offsets), sizes the two device slots for the largest group and creates the
// copy stream and events.  Called at the start of a run; cheap when nothing changed.
int prepare_offload(DinoModule& mod) {
  OffloadState& o = mod.offload;
  if (o.groups.empty()) return 0;
  size_t need = 0;
  for (auto& entry : o.groups) {
    size_t at = 0;
    for (int ci : entry.second.constants) {
      mod.constants[ci].slot_offset = at;
      at += (mod.constants[ci].nbytes + kSlotAlign - 1) / kSlotAlign * kSlotAlign;
    }
    entry.second.bytes = at;
    if (at > need) need = at;
  }
  if (o.copy_stream == nullptr) {
    cudaError_t err = cudaStreamCreateWithFlags(&o.copy_stream, cudaStreamNonBlocking);
    for (int i = 0; i < 2 && err == cudaSuccess; ++i) {
      err = cudaEventCreateWithFlags(&o.ready[i], cudaEventDisableTiming);
      if (err == cudaSuccess) err = cudaEventCreateWithFlags(&o.freed[i], cudaEventDisableTiming);
    }
    if (err != cudaSuccess) return cuda_fail("offload stream / events", err);
  }
  if (need > o.slot_bytes) {
    cudaDeviceSynchronize();                      // nothing may still read or fill the old slots
    for (int i = 0; i < 2; ++i) {
      if (o.slot[i] != nullptr) cudaFree(o.slot[i]);
      o.slot[i] = nullptr;
      const cudaError_t err = cudaMalloc(&o.slot[i], need);
      if (err != cudaSuccess) return cuda_fail("cudaMalloc (offload slot)", err);
      o.resident[i] = -1;
      o.freed_valid[i] = false;
    }
    o.slot_bytes = need;
  }
  return 0;
}

// Copies group g into slot sl on the copy stream, after the last kernel that read the slot.
int issue_upload(DinoModule& mod, int g, int sl) {
  OffloadState& o = mod.offload;
  if (o.freed_valid[sl]) {
    const cudaError_t err = cudaStreamWaitEvent(o.copy_stream, o.freed[sl], 0);
    if (err != cudaSuccess) return cuda_fail("cudaStreamWaitEvent (offload slot free)", err);
  }
  for (int ci : o.groups[g].constants) {
    const ConstantSpec& c = mod.constants[ci];
    const cudaError_t err = cudaMemcpyAsync(static_cast<uint8_t*>(o.slot[sl]) + c.slot_offset, c.host, c.nbytes, cudaMemcpyHostToDevice, o.copy_stream);
    if (err != cudaSuccess) return cuda_fail("cudaMemcpyAsync (offloaded constant)", err);
    ++o.uploads;
    o.upload_bytes += c.nbytes;
  }
  const cudaError_t err = cudaEventRecord(o.ready[sl], o.copy_stream);
  if (err != cudaSuccess) return cuda_fail("cudaEventRecord (offload ready)", err);
  o.resident[sl] = g;
  return 0;
}

// Makes group g available to kernels on `stream`; returns its slot.  `keep` is the slot that must not be overwritten (the
// one the caller is computing from), or -1.
int acquire_group(DinoModule& mod, int g, int keep, cudaStream_t stream, int* slot) {
  OffloadState& o = mod.offload;
  int sl = o.resident[0] == g ? 0 : o.resident[1] == g ? 1 : -1;
  if (sl < 0) {
    sl = keep == 0 ? 1 : keep == 1 ? 0 : (o.resident[0] < 0 ? 0 : o.resident[1] < 0 ? 1 : 0);
    if (int rc = issue_upload(mod, g, sl)) return rc;
  }
  const cudaError_t err = cudaStreamWaitEvent(stream, o.ready[sl], 0);
  if (err != cudaSuccess) return cuda_fail("cudaStreamWaitEvent (offload ready)", err);
  *slot = sl;
  return 0;
}

// cpu_until_first_use: allocate the device buffer and copy the bytes on the run's stream, ahead of the first launch that
// reads them; the constant stays on the device afterwards.
int first_use_upload(ConstantSpec& c, cudaStream_t stream) {
  if (c.host == nullptr) return fail("constant '" + c.name + "' has no host copy to upload");
  cudaError_t err = cudaMalloc(&c.device, c.nbytes);
  if (err != cudaSuccess) return cuda_fail("cudaMalloc (first-use constant)", err);
  err = cudaMemcpyAsync(c.device, c.host, c.nbytes, cudaMemcpyHostToDevice, stream);
  return err == cudaSuccess ? 0 : cuda_fail("cudaMemcpyAsync (first-use constant)", err);
}

void release_offload(DinoModule& mod) {
  OffloadState& o = mod.offload;
  for (int i = 0; i < 2; ++i) {
    if (o.slot[i] != nullptr) cudaFree(o.slot[i]);
    if (o.ready[i] != nullptr) cudaEventDestroy(o.ready[i]);
    if (o.freed[i] != nullptr) cudaEventDestroy(o.freed[i]);
  }
  if (o.copy_stream != nullptr) cudaStreamDestroy(o.copy_stream);
  for (ConstantSpec& c : mod.constants) { c.group = -1; c.policy = residency_policy(c.residency) == RES_DEVICE ? RES_DEVICE : c.policy; }
  mod.offload = OffloadState();
}

bool module_streams_constants(const DinoModule& mod) {
  for (const ConstantSpec& c : mod.constants)
    if (c.policy == RES_OFFLOAD || (c.policy == RES_FIRST_USE && c.device == nullptr)) return true;
  return false;
}

// ---- DINOML_PROFILE_RUN: per-launch event timing -------------------------------------------------------------------
struct ProfileSection { std::string name; int start = -1, end = -1; cudaEvent_t e0 = nullptr, e1 = nullptr; bool started = false, stopped = false; };
int parse_profile_sections(const char* env, std::vector<ProfileSection>* out) {
  const char* cursor = env;
  while (cursor != nullptr && *cursor != '\0') {
    const char* colon = std::strchr(cursor, ':');
    if (colon == nullptr) return fail("DINOML_PROFILE_RUN_SECTIONS entry is missing first ':'");
    char* end1 = nullptr;
    const long a = std::strtol(colon + 1, &end1, 10);
    if (end1 == colon + 1 || *end1 != ':') return fail("DINOML_PROFILE_RUN_SECTIONS entry has invalid start launch");
    char* end2 = nullptr;
    const long b = std::strtol(end1 + 1, &end2, 10);
    if (end2 == end1 + 1) return fail("DINOML_PROFILE_RUN_SECTIONS entry has invalid end launch");
    if (a < 0 || b < a) return fail("DINOML_PROFILE_RUN_SECTIONS requires non-negative start <= end");
    ProfileSection sec;
    sec.name.assign(cursor, size_t(colon - cursor));
    sec.start = int(a);
    sec.end = int(b);
    out->push_back(sec);
    if (*end2 == ',') cursor = end2 + 1;
    else if (*end2 == '\0') cursor = end2;
    else return fail("DINOML_PROFILE_RUN_SECTIONS entries must be comma-separated");
  }
  return 0;
}

// One pass over the plan.  `launch == false` only validates and computes shapes.
int run_plan(DinoSession* s, const DinoTensor* inputs, size_t num_inputs, DinoTensor* outputs, size_t num_outputs,
             bool validate) {
  DinoModule& mod = *s->module;
  if (validate) {
    if (num_inputs != mod.inputs.size()) return fail("dino_session_run expected " + std::to_string(mod.inputs.size()) + " inputs");
    if (num_outputs != mod.outputs.size()) return fail("dino_session_run expected " + std::to_string(mod.outputs.size()) + " outputs");
    if ((num_inputs && inputs == nullptr) || (num_outputs && outputs == nullptr)) return fail("dino_session_run received null tensor arrays");
    for (size_t i = 0; i < num_inputs; ++i)
      if (int rc = check_tensor(mod.tensors[mod.inputs[i]], inputs[i], "input", &s->shapes[mod.inputs[i]])) return rc;
    for (const ConstantSpec& c : mod.constants)
      if (!c.loaded)
        return fail("constant '" + c.name + "' is not loaded" +
                    (!c.encoded ? "" : c.policy == RES_DEVICE ? " (call dino_module_set_encoded_constant)" : " (call dino_module_set_offloaded_encoded_constant)"));
  }
  if (int rc = prepare_offload(mod)) return rc;
  // per-launch timing on request (environment contract of the reference's generated module)
  const bool profile_run = std::getenv("DINOML_PROFILE_RUN") != nullptr;
  const bool profile_verbose = std::getenv("DINOML_PROFILE_RUN_VERBOSE") != nullptr;
  std::vector<ProfileSection> sections;
  if (const char* env = std::getenv("DINOML_PROFILE_RUN_SECTIONS"))
    if (int rc = parse_profile_sections(env, &sections)) return rc;
  for (ProfileSection& sec : sections)
    if (cudaEventCreate(&sec.e0) != cudaSuccess || cudaEventCreate(&sec.e1) != cudaSuccess) return fail("cudaEventCreate failed");
  std::vector<cudaEvent_t> ev0, ev1;
  std::vector<int> ev_node;
  cudaEvent_t total0 = nullptr, total1 = nullptr;
  if (profile_run) {
    if (cudaEventCreate(&total0) != cudaSuccess || cudaEventCreate(&total1) != cudaSuccess) return fail("cudaEventCreate failed");
    cudaEventRecord(total0, s->stream);
  }
  int launch_index = 0, busy_slot = -1;
  std::vector<void*> ptr(mod.tensors.size(), nullptr);
  for (size_t i = 0; i < num_inputs; ++i) ptr[mod.inputs[i]] = tensor_ptr(inputs[i]);
  for (size_t i = 0; i < num_outputs; ++i) ptr[mod.outputs[i]] = outputs[i].data ? tensor_ptr(outputs[i]) : nullptr;
  for (size_t i = 0; i < mod.tensors.size(); ++i) if (mod.tensors[i].role == 2) ptr[i] = s->temps[i];

  for (size_t ni = 0; ni < mod.nodes.size(); ++ni) {
    const NodeSpec& node = mod.nodes[ni];
    ConstantSpec& w = mod.constants[node.b];
    const std::vector<int64_t>& ashape = s->shapes[node.a];
    if (ashape.empty()) return fail("node " + std::to_string(ni) + " consumes a tensor that has no shape yet");
    const int64_t k = ashape.back();
    int64_t m = 1;
    for (size_t i = 0; i + 1 < ashape.size(); ++i) m *= ashape[i];
    if (node.activation != 0 && w.shape[0] % 16 != 0) return fail("dual_gemm_rcr weight must hold 2N rows with N % 8 == 0");
    const int64_t n = node.activation != 0 ? w.shape[0] / 2 : w.shape[0];
    if (k != w.shape[1]) return fail("gemm_rcr K dimension " + std::to_string(k) + " does not match n_per_row " + std::to_string(w.shape[1]));
    if (m > 0x7fffffff || n > 0x7fffffff || k > 0x7fffffff) return fail("gemm_rcr dimension exceeds int range");
    std::vector<int64_t> oshape(ashape.begin(), ashape.end() - 1);
    oshape.push_back(n);
    const TensorSpec& ospec = mod.tensors[node.out];
    if (validate) {
      if (ospec.dtype != mod.tensors[node.a].dtype) return fail("gemm_rcr operands must share one dtype");
      if (ospec.role == 1) {
        size_t oi = 0;
        while (mod.outputs[oi] != node.out) ++oi;
        std::vector<int64_t> given;
        if (int rc = check_tensor(ospec, outputs[oi], "output", &given)) return rc;
        if (given != oshape) return fail("output '" + ospec.name + "' shape does not match the gemm_rcr result shape");
        s->output_shape_valid[oi] = true;
      }
      s->shapes[node.out] = oshape;
    }
    if (m == 0) continue;
    int variant = node.variant;
    for (const DispatchSpec& d : mod.dispatch)
      if (d.node == int(ni) && d.m == m && d.n == n && d.k == k) { variant = d.variant; break; }
    const void* bias = node.bias >= 0 ? mod.constants[node.bias].device : nullptr;
    if (node.bias >= 0 && mod.constants[node.bias].shape.back() != (node.activation != 0 ? 2 * n : n))
      return fail(node.activation != 0 ? "interleaved dual-GEMM bias must hold 2N values" : "bias length does not match N");
    // where the weight bytes are for this launch
    const void* wptr = w.device;
    int slot = -1;
    if (w.policy == RES_FIRST_USE && w.device == nullptr) {
      if (int rc = first_use_upload(w, s->stream)) return rc;
      wptr = w.device;
    } else if (w.policy == RES_OFFLOAD) {
      if (int rc = acquire_group(mod, w.group, busy_slot, s->stream, &slot)) return rc;
      wptr = static_cast<const uint8_t*>(mod.offload.slot[slot]) + w.slot_offset;
      busy_slot = slot;
    }
    for (ProfileSection& sec : sections)
      if (sec.start == launch_index) { cudaEventRecord(sec.e0, s->stream); sec.started = true; }
    if (profile_run) {
      cudaEvent_t a = nullptr, b = nullptr;
      if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) return fail("cudaEventCreate failed");
      ev0.push_back(a); ev1.push_back(b); ev_node.push_back(int(ni));
      cudaEventRecord(a, s->stream);
    }
    const int rc = node.activation != 0
                       ? b200gguf::dual_gemm_rcr(ptr[node.a], wptr, bias, ptr[node.out], w.qtype, ospec.dtype, int(m), int(n), int(k),
                                                 node.activation, variant, s->stream)
                       : b200gguf::gemm_rcr(ptr[node.a], wptr, bias, ptr[node.out], w.qtype, ospec.dtype, int(m), int(n), int(k),
                                            variant, s->stream);
    if (profile_run) cudaEventRecord(ev1.back(), s->stream);
    for (ProfileSection& sec : sections)
      if (sec.end == launch_index) { cudaEventRecord(sec.e1, s->stream); sec.stopped = true; }
    ++launch_index;
    if (slot >= 0 && rc == 0) {
      // the slot is free again once this launch has read it; then stream the next group into the other slot while this
      // one computes
      OffloadState& o = mod.offload;
      cudaEventRecord(o.freed[slot], s->stream);
      o.freed_valid[slot] = true;
      for (size_t nj = ni + 1; nj < mod.nodes.size(); ++nj) {
        const ConstantSpec& nw = mod.constants[mod.nodes[nj].b];
        if (nw.policy != RES_OFFLOAD || nw.group == w.group) continue;
        if (o.resident[0] != nw.group && o.resident[1] != nw.group)
          if (int rc2 = issue_upload(mod, nw.group, slot ^ 1)) return rc2;
        break;
      }
    }
    if (rc != 0) {
      static const char* const kText[] = {"ok", "null pointer", "non-positive dimension", "k not a multiple of the block",
                                          "CUDA launch failed", "unsupported qtype", "unsupported dtype", "alignment",
                                          "shape outside variant range", "device wait gave up"};
      std::string why = rc < 10 ? kText[rc] : "error";
      if (rc == 4) why += std::string(" (") + cudaGetErrorString(cudaPeekAtLastError()) + ")";
      return fail("gemm_rcr node " + std::to_string(ni) + " (m=" + std::to_string(m) + ", n=" + std::to_string(n) + ", k=" + std::to_string(k) +
                  ", variant " + std::to_string(variant) + ") failed: " + why);
    }
  }
  if (profile_run || !sections.empty()) {
    if (profile_run) cudaEventRecord(total1, s->stream);
    if (cudaStreamSynchronize(s->stream) != cudaSuccess) return fail("profile run: stream synchronize failed");
    if (profile_run) {
      double op_ms[3] = {0, 0, 0};
      size_t op_count[3] = {0, 0, 0};
      static const char* const kOp[3] = {"gemm_rcr", "dual_gemm_rcr_silu", "dual_gemm_rcr_fast_gelu"};
      for (size_t i = 0; i < ev0.size(); ++i) {
        float ms = 0.f;
        cudaEventElapsedTime(&ms, ev0[i], ev1[i]);
        const NodeSpec& node = mod.nodes[ev_node[i]];
        op_ms[node.activation] += ms;
        ++op_count[node.activation];
        if (profile_verbose)
          std::fprintf(stderr, "[dinoml_profile_launch] label=node%d:%s:%s ms=%.6f\n", ev_node[i], kOp[node.activation],
                       mod.tensors[node.out].name.c_str(), double(ms));
        cudaEventDestroy(ev0[i]);
        cudaEventDestroy(ev1[i]);
      }
      float total = 0.f;
      cudaEventElapsedTime(&total, total0, total1);
      std::fprintf(stderr, "[dinoml_profile] total_gpu_ms=%.6f\n", double(total));
      for (int op = 0; op < 3; ++op)
        if (op_count[op] != 0)
          std::fprintf(stderr, "[dinoml_profile] op=%s count=%zu total_ms=%.6f mean_ms=%.6f\n", kOp[op], op_count[op], op_ms[op],
                       op_ms[op] / double(op_count[op]));
      cudaEventDestroy(total0);
      cudaEventDestroy(total1);
    }
    for (ProfileSection& sec : sections) {
      if (!sec.started || !sec.stopped) return fail("DINOML_PROFILE_RUN_SECTIONS range did not match generated launch indices");
      float ms = 0.f;
      cudaEventElapsedTime(&ms, sec.e0, sec.e1);
      std::fprintf(stderr, "[dinoml_profile_section] name=%s start=%d end=%d ms=%.6f\n", sec.name.c_str(), sec.start, sec.end, double(ms));
      cudaEventDestroy(sec.e0);
      cudaEventDestroy(sec.e1);
    }
    std::fflush(stderr);
  }
  return 0;
}

}  // namespace

extern "C" {

int dino_runtime_fail(const char* message) { return fail(message ? message : "unknown error"); }
int dino_abi_version(void) { return DINO_RUNTIME_ABI_VERSION; }

int dino_device_malloc(void** out, size_t nbytes) {
  if (out == nullptr) return fail("dino_device_malloc received null pointer");
  const cudaError_t err = cudaMalloc(out, nbytes);
  return err == cudaSuccess ? 0 : cuda_fail("cudaMalloc", err);
}
int dino_device_free(void* ptr) {
  const cudaError_t err = cudaFree(ptr);
  return err == cudaSuccess ? 0 : cuda_fail("cudaFree", err);
}
int dino_copy_host_to_device(void* dst, const void* src, size_t nbytes) {
  const cudaError_t err = cudaMemcpy(dst, src, nbytes, cudaMemcpyHostToDevice);
  return err == cudaSuccess ? 0 : cuda_fail("cudaMemcpy H2D", err);
}
int dino_copy_device_to_host(void* dst, const void* src, size_t nbytes) {
  const cudaError_t err = cudaMemcpy(dst, src, nbytes, cudaMemcpyDeviceToHost);
  return err == cudaSuccess ? 0 : cuda_fail("cudaMemcpy D2H", err);
}
int dino_copy_device_to_device(void* dst, const void* src, size_t nbytes) {
  const cudaError_t err = cudaMemcpy(dst, src, nbytes, cudaMemcpyDeviceToDevice);
  return err == cudaSuccess ? 0 : cuda_fail("cudaMemcpy D2D", err);
}

int dino_module_load(const char* artifact_dir, DinoModule** out) { return load_module(artifact_dir, true, out); }
int dino_module_load_deferred(const char* artifact_dir, DinoModule** out) { return load_module(artifact_dir, false, out); }

int dino_module_load_constants(DinoModule* module, const char* constants_path) {
  if (module == nullptr || constants_path == nullptr) return fail("dino_module_load_constants received null pointer");
  std::ifstream in(constants_path, std::ios::binary);
  if (!in) return fail(std::string("cannot open ") + constants_path);
  std::vector<char> staging;
  for (ConstantSpec& c : module->constants) {
    if (c.encoded && c.residency == "manual_runtime_load") continue;   // uploaded by dino_module_set_encoded_constant
    if (c.encoded && residency_policy(c.residency) != RES_DEVICE) continue;   // registered by dino_module_set_offloaded_encoded_constant
    staging.resize(c.nbytes);
    in.seekg(std::streamoff(c.offset));
    if (!in.read(staging.data(), std::streamsize(c.nbytes))) return fail("constants file is too short for '" + c.name + "'");
    if (int rc = ensure_constant_buffer(c)) return rc;
    const cudaError_t err = cudaMemcpy(c.device, staging.data(), c.nbytes, cudaMemcpyHostToDevice);
    if (err != cudaSuccess) return cuda_fail("cudaMemcpy (constant)", err);
    c.loaded = true;
  }
  return 0;
}

int dino_module_unload_constants(DinoModule* module) {
  if (module == nullptr) return fail("dino_module_unload_constants received null pointer");
  cudaDeviceSynchronize();
  for (ConstantSpec& c : module->constants) {
    if (c.device != nullptr) cudaFree(c.device);
    if (c.host != nullptr) cudaFreeHost(c.host);
    c.device = nullptr;
    c.host = nullptr;
    c.loaded = false;
  }
  release_offload(*module);
  ++module->generation;
  return 0;
}

int dino_module_set_constant(DinoModule* module, const char* name, const DinoTensor* tensor) {
  if (module == nullptr || name == nullptr || tensor == nullptr) return fail("dino_module_set_constant received null pointer");
  const int idx = find_constant(*module, name);
  if (idx < 0) return fail(std::string("unknown constant '") + name + "'");
  ConstantSpec& c = module->constants[idx];
  if (c.encoded) return fail(std::string("constant '") + name + "' is GGUF-encoded; use dino_module_set_encoded_constant");
  if (tensor->data == nullptr || tensor->shape == nullptr) return fail("dino_module_set_constant tensor has null data or shape");
  if (tensor->dtype != c.dtype || tensor->ndim != c.shape.size()) return fail(std::string("constant '") + name + "' dtype/rank mismatch");
  for (size_t i = 0; i < tensor->ndim; ++i)
    if (tensor->shape[i] != c.shape[i]) return fail(std::string("constant '") + name + "' shape mismatch");
  if (tensor->device_type != DINO_DEVICE_CUDA) return fail("dino_module_set_constant expects a CUDA tensor");
  if (int rc = ensure_constant_buffer(c)) return rc;
  const cudaError_t err = cudaMemcpy(c.device, tensor_ptr(*tensor), c.nbytes, cudaMemcpyDeviceToDevice);
  if (err != cudaSuccess) return cuda_fail("cudaMemcpy (set_constant)", err);
  c.loaded = true;
  return 0;
}

int dino_module_set_encoded_constant(DinoModule* module, const char* name, const void* device_bytes, size_t nbytes) {
  if (module == nullptr || name == nullptr || device_bytes == nullptr) return fail("dino_module_set_encoded_constant received null pointer");
  const int idx = find_constant(*module, name);
  if (idx < 0) return fail(std::string("unknown constant '") + name + "'");
  ConstantSpec& c = module->constants[idx];
  if (!c.encoded) return fail(std::string("constant '") + name + "' is not GGUF-encoded");
  if (nbytes != c.nbytes)
    return fail(std::string("constant '") + name + "' expects exactly " + std::to_string(c.nbytes) + " encoded bytes, got " + std::to_string(nbytes));
  if (int rc = ensure_constant_buffer(c)) return rc;
  const cudaError_t err = cudaMemcpy(c.device, device_bytes, nbytes, cudaMemcpyDeviceToDevice);
  if (err != cudaSuccess) return cuda_fail("cudaMemcpy (set_encoded_constant)", err);
  c.loaded = true;
  return 0;
}

int dino_module_free(DinoModule* module) {
  if (module == nullptr) return 0;
  cudaDeviceSynchronize();
  for (ConstantSpec& c : module->constants) {
    if (c.device != nullptr) cudaFree(c.device);
    if (c.host != nullptr) cudaFreeHost(c.host);
  }
  release_offload(*module);
  delete module;
  return 0;
}

int dino_module_set_offloaded_encoded_constant(DinoModule* module, const char* name, const void* host_bytes, size_t nbytes, int group) {
  if (module == nullptr || name == nullptr || host_bytes == nullptr) return fail("dino_module_set_offloaded_encoded_constant received null pointer");
  const int idx = find_constant(*module, name);
  if (idx < 0) return fail(std::string("unknown constant '") + name + "'");
  ConstantSpec& c = module->constants[idx];
  if (!c.encoded) return fail(std::string("constant '") + name + "' is not GGUF-encoded");
  const int policy = residency_policy(c.residency);
  if (policy == RES_DEVICE)
    return fail(std::string("constant '") + name + "' has residency " + c.residency + ": it lives on the device (use dino_module_set_encoded_constant)");
  if (nbytes != c.nbytes)
    return fail(std::string("constant '") + name + "' expects exactly " + std::to_string(c.nbytes) + " encoded bytes, got " + std::to_string(nbytes));
  if (policy == RES_OFFLOAD && group < 0) return fail("offload group must be non-negative");
  if (c.host == nullptr) {
    const cudaError_t err = cudaMallocHost(&c.host, nbytes);
    if (err != cudaSuccess) return cuda_fail("cudaMallocHost (host-resident constant)", err);
    module->offload.host_bytes += nbytes;
  }
  std::memcpy(c.host, host_bytes, nbytes);
  if (c.device != nullptr) {            // a first-use constant that was already uploaded: refresh the device copy too
    const cudaError_t err = cudaMemcpy(c.device, c.host, nbytes, cudaMemcpyHostToDevice);
    if (err != cudaSuccess) return cuda_fail("cudaMemcpy (first-use constant refresh)", err);
  }
  if (policy == RES_OFFLOAD) {
    OffloadState& o = module->offload;
    if (c.group >= 0 && c.group != group) return fail(std::string("constant '") + name + "' is already in offload group " + std::to_string(c.group));
    if (c.group < 0) {
      c.group = group;
      o.groups[group].constants.push_back(idx);
    }
    for (int i = 0; i < 2; ++i)
      if (o.resident[i] == group) o.resident[i] = -1;      // the slot image of this group is stale
  }
  c.policy = policy;
  c.loaded = true;
  return 0;
}

int dino_module_get_residency_stats(DinoModule* module, size_t* device_resident_bytes, size_t* device_slot_bytes, size_t* pinned_host_bytes,
                                    size_t* uploads, size_t* upload_bytes) {
  if (module == nullptr) return fail("dino_module_get_residency_stats received null pointer");
  size_t resident = 0;
  for (const ConstantSpec& c : module->constants) if (c.encoded && c.device != nullptr) resident += c.nbytes;
  if (device_resident_bytes) *device_resident_bytes = resident;
  if (device_slot_bytes) *device_slot_bytes = 2 * module->offload.slot_bytes;
  if (pinned_host_bytes) *pinned_host_bytes = module->offload.host_bytes;
  if (uploads) *uploads = module->offload.uploads;
  if (upload_bytes) *upload_bytes = module->offload.upload_bytes;
  return 0;
}

const char* dino_module_get_metadata_json(DinoModule* module) { return module ? module->metadata_json.c_str() : ""; }

int dino_session_create(DinoModule* module, DinoSession** out) {
  if (module == nullptr || out == nullptr) return fail("dino_session_create received null pointer");
  *out = nullptr;
  DinoSession* s = new DinoSession();
  s->module = module;
  cudaError_t err = cudaStreamCreateWithFlags(&s->owned_stream, cudaStreamNonBlocking);
  if (err != cudaSuccess) { delete s; return cuda_fail("cudaStreamCreateWithFlags", err); }
  s->stream = s->owned_stream;
  s->temps.assign(module->tensors.size(), nullptr);
  s->shapes.assign(module->tensors.size(), {});
  s->output_shape_valid.assign(module->outputs.size(), false);
  for (size_t i = 0; i < module->tensors.size(); ++i) {
    if (module->tensors[i].role != 2) continue;
    err = cudaMalloc(&s->temps[i], module->tensors[i].max_bytes());
    if (err != cudaSuccess) { dino_session_destroy(s); return cuda_fail("cudaMalloc (session temporary)", err); }
  }
  *out = s;
  return 0;
}

int dino_session_destroy(DinoSession* session) {
  if (session == nullptr) return 0;
  if (session->owned_stream != nullptr) {
    cudaStreamSynchronize(session->owned_stream);
    cudaStreamDestroy(session->owned_stream);
  }
  for (auto& entry : session->graphs)
    if (entry.second.exec != nullptr) cudaGraphExecDestroy(entry.second.exec);
  for (void* p : session->temps) if (p != nullptr) cudaFree(p);
  delete session;
  return 0;
}

int dino_session_set_stream(DinoSession* session, void* stream) {
  if (session == nullptr) return fail("dino_session_set_stream received null pointer");
  session->external_stream = stream != nullptr;
  session->stream = stream != nullptr ? static_cast<cudaStream_t>(stream) : session->owned_stream;
  return 0;
}

int dino_session_get_output_shape(DinoSession* session, size_t output_index, int64_t* out_shape, size_t* inout_ndim) {
  if (session == nullptr || inout_ndim == nullptr) return fail("dino_session_get_output_shape received null pointer");
  if (output_index >= session->module->outputs.size()) return fail("output index out of range");
  if (!session->output_shape_valid[output_index]) return fail("output shape is not available before the first run");
  const std::vector<int64_t>& shape = session->shapes[session->module->outputs[output_index]];
  if (out_shape == nullptr || *inout_ndim < shape.size()) { *inout_ndim = shape.size(); return out_shape == nullptr ? 0 : fail("output shape buffer too small"); }
  std::memcpy(out_shape, shape.data(), shape.size() * sizeof(int64_t));
  *inout_ndim = shape.size();
  return 0;
}

// The three optional session entries of the reference's generated module.  This runtime keeps no per-session temporary arena
// (the fused kernels need no dense scratch) and the quantized-linear graphs have no state tensors, so the arena calls
// validate their arguments and succeed, and no state index is valid.
int dino_session_set_temp_arena_policy(DinoSession* session, int policy) {
  if (session == nullptr) return fail("dino_session_set_temp_arena_policy received null session");
  if (policy < 0 || policy > 2) return fail("Unsupported temp arena allocation policy");
  return 0;
}
int dino_session_release_temp_arena(DinoSession* session) {
  if (session == nullptr) return fail("dino_session_release_temp_arena received null session");
  return 0;
}
int dino_session_get_state_pointer(DinoSession* session, size_t state_index, void** out_data) {
  (void)state_index;
  if (session == nullptr || out_data == nullptr) return fail("dino_session_get_state_pointer received null argument");
  return fail("dino_session_get_state_pointer received invalid state index");
}

int dino_session_set_graph_replay(DinoSession* session, int enabled) {
  if (session == nullptr) return fail("dino_session_set_graph_replay received null pointer");
  session->graph_replay = enabled != 0;
  return 0;
}

int dino_session_get_graph_stats(DinoSession* session, size_t* cached_graphs, size_t* graph_launches) {
  if (session == nullptr) return fail("dino_session_get_graph_stats received null pointer");
  size_t n = 0;
  for (const auto& entry : session->graphs) n += entry.second.exec != nullptr ? 1 : 0;
  if (cached_graphs) *cached_graphs = n;
  if (graph_launches) *graph_launches = session->graph_launches;
  return 0;
}

// Steady-state path of dino_session_run: the launch sequence of one (input shapes, input / output pointers) combination is
// captured the second time it is seen and replayed afterwards; validation ran when it was captured.  Returns 1 if the
// call was served (rc in *rc_out), 0 if the caller should run the plan the ordinary way.
static int run_replayed(DinoSession* s, const DinoTensor* inputs, size_t num_inputs, DinoTensor* outputs, size_t num_outputs, int* rc_out) {
  DinoModule& mod = *s->module;
  if (!s->graph_replay || module_streams_constants(mod) || std::getenv("DINOML_PROFILE_RUN") != nullptr ||
      std::getenv("DINOML_PROFILE_RUN_SECTIONS") != nullptr)
    return 0;
  if (num_inputs != mod.inputs.size() || num_outputs != mod.outputs.size() || (num_inputs && !inputs) || (num_outputs && !outputs)) return 0;
  if (s->graph_generation != mod.generation) {             // constant buffers were released since: every captured pointer is stale
    for (auto& entry : s->graphs) if (entry.second.exec != nullptr) cudaGraphExecDestroy(entry.second.exec);
    s->graphs.clear();
    s->graph_generation = mod.generation;
  }
  std::vector<int64_t> key;
  for (size_t i = 0; i < num_inputs; ++i) {
    if (inputs[i].shape == nullptr || inputs[i].data == nullptr) return 0;
    key.push_back(int64_t(reinterpret_cast<intptr_t>(tensor_ptr(inputs[i]))));
    key.push_back(int64_t(inputs[i].ndim));
    key.insert(key.end(), inputs[i].shape, inputs[i].shape + inputs[i].ndim);
  }
  for (size_t i = 0; i < num_outputs; ++i) {
    if (outputs[i].data == nullptr) return 0;
    key.push_back(int64_t(reinterpret_cast<intptr_t>(tensor_ptr(outputs[i]))));
  }
  if (s->graphs.size() > 64 && s->graphs.find(key) == s->graphs.end()) {     // callers that pass ever-changing buffers: start over
    for (auto& entry : s->graphs) if (entry.second.exec != nullptr) cudaGraphExecDestroy(entry.second.exec);
    s->graphs.clear();
  }
  DinoSession::CachedGraph& cg = s->graphs[key];
  if (cg.exec != nullptr) {
    s->shapes = cg.out_shapes;
    std::fill(s->output_shape_valid.begin(), s->output_shape_valid.end(), true);
    const cudaError_t err = cudaGraphLaunch(cg.exec, s->stream);
    ++s->graph_launches;
    *rc_out = err == cudaSuccess ? 0 : cuda_fail("cudaGraphLaunch", err);
    return 1;
  }
  if (cg.seen < 1) {                 // not yet run successfully the ordinary way (or a capture failed before): ordinary run
    if (cg.seen == 0) s->pending_key = key;
    return 0;
  }
  // seen once, and that run succeeded (every lazily created workspace of the kernels exists): capture this one
  cudaGraph_t graph = nullptr;
  if (cudaStreamBeginCapture(s->stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) { cudaGetLastError(); cg.seen = -1; return 0; }
  const int rc = run_plan(s, inputs, num_inputs, outputs, num_outputs, true);
  const bool ended = cudaStreamEndCapture(s->stream, &graph) == cudaSuccess && graph != nullptr;
  bool ok = rc == 0 && ended && cudaGraphInstantiate(&cg.exec, graph, 0) == cudaSuccess;
  if (graph) cudaGraphDestroy(graph);
  if (!ok) {                         // nothing was launched: forget the capture and let the caller run the plan directly
    cudaGetLastError();
    cg.exec = nullptr;
    cg.seen = -1;
    return 0;
  }
  cg.out_shapes = s->shapes;
  const cudaError_t err = cudaGraphLaunch(cg.exec, s->stream);
  ++s->graph_launches;
  *rc_out = err == cudaSuccess ? 0 : cuda_fail("cudaGraphLaunch", err);
  return 1;
}

// A combination counts as seen once a run of it has succeeded the ordinary way.
static void note_ordinary_run(DinoSession* s) {
  if (s->pending_key.empty()) return;
  auto it = s->graphs.find(s->pending_key);
  if (it != s->graphs.end() && it->second.seen == 0) it->second.seen = 1;
  s->pending_key.clear();
}

int dino_session_run(DinoSession* session, const DinoTensor* inputs, size_t num_inputs, DinoTensor* outputs, size_t num_outputs) {
  if (session == nullptr) return fail("dino_session_run received null session");
  int replay_rc = 0;
  session->pending_key.clear();
  if (run_replayed(session, inputs, num_inputs, outputs, num_outputs, &replay_rc)) {
    if (replay_rc != 0) return replay_rc;
  } else if (int rc = run_plan(session, inputs, num_inputs, outputs, num_outputs, true)) {
    return rc;
  } else {
    note_ordinary_run(session);
  }
  if (!session->external_stream) {
    const cudaError_t err = cudaStreamSynchronize(session->stream);
    if (err != cudaSuccess) return cuda_fail("dino_session_run synchronize", err);
  }
  return 0;
}

int dino_session_run_staged(DinoSession* session, const void* host_in, void* device_in, size_t in_bytes, const DinoTensor* inputs,
                            size_t num_inputs, DinoTensor* outputs, size_t num_outputs, const void* device_out, void* host_out,
                            size_t out_bytes) {
  if (session == nullptr) return fail("dino_session_run_staged received null session");
  if ((in_bytes && (host_in == nullptr || device_in == nullptr)) || (out_bytes && (host_out == nullptr || device_out == nullptr)))
    return fail("dino_session_run_staged received a null staging buffer");
  cudaStream_t stream = session->stream;
  if (in_bytes) {
    const cudaError_t err = cudaMemcpyAsync(device_in, host_in, in_bytes, cudaMemcpyHostToDevice, stream);
    if (err != cudaSuccess) return cuda_fail("cudaMemcpyAsync (staged inputs)", err);
  }
  int replay_rc = 0;
  session->pending_key.clear();
  if (run_replayed(session, inputs, num_inputs, outputs, num_outputs, &replay_rc)) {
    if (replay_rc != 0) return replay_rc;
  } else if (int rc = run_plan(session, inputs, num_inputs, outputs, num_outputs, true)) {
    return rc;
  } else {
    note_ordinary_run(session);
  }
  if (out_bytes) {
    const cudaError_t err = cudaMemcpyAsync(host_out, device_out, out_bytes, cudaMemcpyDeviceToHost, stream);
    if (err != cudaSuccess) return cuda_fail("cudaMemcpyAsync (staged outputs)", err);
  }
  const cudaError_t err = cudaStreamSynchronize(stream);
  return err == cudaSuccess ? 0 : cuda_fail("dino_session_run_staged synchronize", err);
}

int dino_session_run_staged_on(DinoSession* session, void* stream, int graph_replay, const void* host_in, void* device_in, size_t in_bytes,
                               const DinoTensor* inputs, size_t num_inputs, DinoTensor* outputs, size_t num_outputs,
                               const void* device_out, void* host_out, size_t out_bytes) {
  if (session == nullptr) return fail("dino_session_run_staged_on received null session");
  // this call's stream and replay setting; the session's own come back afterwards, whatever the outcome
  const cudaStream_t saved_stream = session->stream;
  const bool saved_external = session->external_stream, saved_replay = session->graph_replay;
  if (stream != nullptr) { session->stream = static_cast<cudaStream_t>(stream); session->external_stream = true; }
  session->graph_replay = graph_replay != 0;
  const int rc = dino_session_run_staged(session, host_in, device_in, in_bytes, inputs, num_inputs, outputs, num_outputs, device_out, host_out,
                                         out_bytes);
  session->stream = saved_stream;
  session->external_stream = saved_external;
  session->graph_replay = saved_replay;
  return rc;
}

// float32 <-> bfloat16 bit patterns on the host, for callers whose arrays are float32 (numpy has no bfloat16): round to
// nearest even exactly as the reference's Python does (src/dinoml/ir.py:68-73: bits + 0x7FFF + lsb, high half), NaN kept
// a NaN; widening is the 16 bits followed by 16 zeros.
// Written on 32-bit integer views with no call in the loop body so that the host compiler vectorizes them (an 11008-element
// result widens in 0.4 us instead of 3 us).
typedef uint32_t __attribute__((may_alias)) aliased_u32;
void dino_convert_f32_to_bf16(const float* src, uint16_t* dst, size_t count) {
  const aliased_u32* __restrict__ in = reinterpret_cast<const aliased_u32*>(src);
  uint16_t* __restrict__ out = dst;
  for (size_t i = 0; i < count; ++i) {
    const uint32_t bits = in[i];
    out[i] = uint16_t((bits + 0x7FFFu + ((bits >> 16) & 1u)) >> 16);
  }
}
void dino_convert_bf16_to_f32(const uint16_t* src, float* dst, size_t count) {
  size_t i = 0;
#if defined(__SSE2__)
  // 8 values per step: interleaving with zeros puts each 16-bit pattern into the high half of a 32-bit lane
  const __m128i zero = _mm_setzero_si128();
  for (; i + 8 <= count; i += 8) {
    const __m128i v = _mm_loadu_si128(reinterpret_cast<const __m128i*>(src + i));
    _mm_storeu_si128(reinterpret_cast<__m128i*>(dst + i), _mm_unpacklo_epi16(zero, v));
    _mm_storeu_si128(reinterpret_cast<__m128i*>(dst + i + 4), _mm_unpackhi_epi16(zero, v));
  }
#endif
  aliased_u32* out = reinterpret_cast<aliased_u32*>(dst);
  for (; i < count; ++i) out[i] = uint32_t(src[i]) << 16;
}

int dino_session_benchmark(DinoSession* session, const DinoTensor* inputs, size_t num_inputs, DinoTensor* outputs,
                           size_t num_outputs, size_t warmup_runs, size_t measured_runs, double* out_elapsed_ms,
                           size_t out_elapsed_count) {
  if (session == nullptr) return fail("dino_session_benchmark received null session");
  if (measured_runs == 0 || out_elapsed_ms == nullptr || out_elapsed_count < measured_runs)
    return fail("dino_session_benchmark needs measured_runs > 0 and an output array of at least that length");
  if (int rc = run_plan(session, inputs, num_inputs, outputs, num_outputs, true)) return rc;   // validates + first warm run
  for (size_t i = 1; i < warmup_runs; ++i)
    if (int rc = run_plan(session, inputs, num_inputs, outputs, num_outputs, false)) return rc;
  cudaError_t err = cudaStreamSynchronize(session->stream);
  if (err != cudaSuccess) return cuda_fail("dino_session_benchmark warm-up", err);

  // Graph replay on the owned stream (skipped on an external stream, as the reference does); set
  // DINOML_REQUIRE_BENCHMARK_GRAPH to turn a capture failure into an error instead of direct launches.
  cudaGraphExec_t exec = nullptr;
  if (!session->external_stream && !module_streams_constants(*session->module)) {   // weights streamed from the host: direct launches
    cudaGraph_t graph = nullptr;
    bool ok = cudaStreamBeginCapture(session->stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
    if (ok) {
      const int rc = run_plan(session, inputs, num_inputs, outputs, num_outputs, false);
      ok = cudaStreamEndCapture(session->stream, &graph) == cudaSuccess && rc == 0 && graph != nullptr;
    }
    if (ok) ok = cudaGraphInstantiate(&exec, graph, 0) == cudaSuccess;
    if (graph != nullptr) cudaGraphDestroy(graph);
    if (!ok) {
      exec = nullptr;
      cudaGetLastError();
      if (std::getenv("DINOML_REQUIRE_BENCHMARK_GRAPH") != nullptr) return fail("dino_session_benchmark could not capture a CUDA graph");
    }
  }
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return fail("cudaEventCreate failed");
  int rc = 0;
  for (size_t i = 0; i < measured_runs && rc == 0; ++i) {
    cudaEventRecord(e0, session->stream);
    if (exec != nullptr) {
      if (cudaGraphLaunch(exec, session->stream) != cudaSuccess) rc = fail("cudaGraphLaunch failed");
    } else {
      rc = run_plan(session, inputs, num_inputs, outputs, num_outputs, false);
    }
    cudaEventRecord(e1, session->stream);
    if (rc == 0 && cudaEventSynchronize(e1) != cudaSuccess) rc = fail("cudaEventSynchronize failed");
    float ms = 0.f;
    if (rc == 0 && cudaEventElapsedTime(&ms, e0, e1) != cudaSuccess) rc = fail("cudaEventElapsedTime failed");
    out_elapsed_ms[i] = double(ms);
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (exec != nullptr) cudaGraphExecDestroy(exec);
  return rc;
}

}  // extern "C"
