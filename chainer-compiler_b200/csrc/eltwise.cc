// Fused elementwise groups: source generator (the counterpart of BuildNvrtcProgram,
// compiler/nvrtc_builder.cc:91-206) and the ElementWiseNvrtc op body (runtime/ops/nvrtc.cc:90-161).
//
// Differences from the reference, all deliberate:
//  * the generated kernel is single-pass, grid-stride and moves 128 bits per load/store (the
//    reference's is one scalar element per thread, 128 threads per block, built for compute_50);
//  * a second, scalar kernel `fusion<id>_s` is emitted for buffers that are not 16-byte aligned;
//  * Sigmoid is 1/(1+exp(-x)) (good relative accuracy for very negative x) instead of
//    tanh(x/2)/2+1/2 (nvrtc_builder.cc:133-136), and constants are printed with full precision
//    instead of the stream default of 6 significant digits (:183);
//  * fp16 groups compute in fp32 and round once on store;
//  * compilation targets sm_100a and yields a cubin; the cache is guarded by a mutex.
#include <cuda.h>
#include <dlfcn.h>
#include <string.h>

#include <map>
#include <mutex>
#include <queue>
#include <set>
#include <sstream>
#include <string>
#include <vector>

#include "common.h"

namespace chxq {
namespace {

std::string cleanse(const std::string& s, const char* prefix) {
    std::string o = prefix;
    for (char c : s) o += (isalnum(static_cast<unsigned char>(c)) ? c : '_');
    return o;
}

const char* op_comment(int op) {
    switch (op) {
        case CHXQ_EW_IDENTITY: return "Identity";
        case CHXQ_EW_TANH: return "Tanh";
        case CHXQ_EW_EXP: return "Exp";
        case CHXQ_EW_SIGMOID: return "Sigmoid";
        case CHXQ_EW_ADD: return "Add";
        case CHXQ_EW_SUB: return "Sub";
        case CHXQ_EW_MUL: return "Mul";
        case CHXQ_EW_DIV: return "Div";
        case CHXQ_EW_CONSTANT: return "Constant";
    }
    return "?";
}

int n_operands(int op) {
    if (op == CHXQ_EW_CONSTANT) return 0;
    if (op >= CHXQ_EW_ADD && op <= CHXQ_EW_DIV) return 2;
    return 1;
}

// ---------------------------------------------------------------------------------------------
// NVRTC and driver entry points, resolved at run time so that the library loads on a host without
// a GPU (the build check) and fails with a clear message when the JIT pieces are missing.
// ---------------------------------------------------------------------------------------------
typedef struct _nvrtcProgram* nvrtcProgram;
struct Nvrtc {
    int (*CreateProgram)(nvrtcProgram*, const char*, const char*, int, const char* const*, const char* const*);
    int (*CompileProgram)(nvrtcProgram, int, const char* const*);
    int (*GetProgramLogSize)(nvrtcProgram, size_t*);
    int (*GetProgramLog)(nvrtcProgram, char*);
    int (*GetCUBINSize)(nvrtcProgram, size_t*);
    int (*GetCUBIN)(nvrtcProgram, char*);
    int (*DestroyProgram)(nvrtcProgram*);
    const char* (*GetErrorString)(int);
    bool ok = false;
    std::string why;
};

Nvrtc& nvrtc() {
    static Nvrtc n;
    static std::once_flag once;
    std::call_once(once, [] {
        std::vector<std::string> names;
        if (const char* env = getenv("CHXQ_NVRTC_PATH")) names.push_back(env);
        names.push_back("libnvrtc.so.12");
        names.push_back("/usr/local/cuda/lib64/libnvrtc.so.12");
        names.push_back("libnvrtc.so");
        void* h = nullptr;
        for (const auto& nm : names) {
            h = dlopen(nm.c_str(), RTLD_NOW | RTLD_LOCAL);
            if (h) break;
        }
        if (!h) {
            n.why = "libnvrtc.so.12 could not be loaded (set CHXQ_NVRTC_PATH)";
            return;
        }
#define LOAD(field, sym)                                            \
    n.field = reinterpret_cast<decltype(n.field)>(dlsym(h, sym));   \
    if (!n.field) {                                                 \
        n.why = std::string("libnvrtc lacks ") + sym;               \
        return;                                                     \
    }
        LOAD(CreateProgram, "nvrtcCreateProgram");
        LOAD(CompileProgram, "nvrtcCompileProgram");
        LOAD(GetProgramLogSize, "nvrtcGetProgramLogSize");
        LOAD(GetProgramLog, "nvrtcGetProgramLog");
        LOAD(GetCUBINSize, "nvrtcGetCUBINSize");
        LOAD(GetCUBIN, "nvrtcGetCUBIN");
        LOAD(DestroyProgram, "nvrtcDestroyProgram");
        LOAD(GetErrorString, "nvrtcGetErrorString");
#undef LOAD
        n.ok = true;
    });
    return n;
}

struct Driver {
    CUresult (*ModuleLoadData)(CUmodule*, const void*);
    CUresult (*ModuleGetFunction)(CUfunction*, CUmodule, const char*);
    CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream, void**, void**);
    bool ok = false;
    std::string why;
};

Driver& driver() {
    static Driver d;
    static std::once_flag once;
    std::call_once(once, [] {
        auto get = [](const char* sym, void** out) {
            cudaDriverEntryPointQueryResult q;
            if (cudaGetDriverEntryPoint(sym, out, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) {
                cudaGetLastError();
                return false;
            }
            return true;
        };
        if (!get("cuModuleLoadData", reinterpret_cast<void**>(&d.ModuleLoadData)) ||
            !get("cuModuleGetFunction", reinterpret_cast<void**>(&d.ModuleGetFunction)) ||
            !get("cuLaunchKernel", reinterpret_cast<void**>(&d.LaunchKernel))) {
            d.why = "CUDA driver entry points (cuModuleLoadData, cuModuleGetFunction, cuLaunchKernel) are unavailable";
            return;
        }
        d.ok = true;
    });
    return d;
}

struct Loaded {
    CUfunction vec;
    CUfunction scalar;
};

std::mutex g_cache_mu;
std::map<std::pair<int, std::string>, Loaded> g_cache;  // (device, source text) -> functions

int compile_and_load(const std::string& code, int fusion_id, Loaded* out) {
    int dev = 0;
    CHXQ_CUDA(cudaGetDevice(&dev));
    CHXQ_CUDA(cudaFree(0));  // make sure the primary context exists and is current
    std::lock_guard<std::mutex> lock(g_cache_mu);
    auto key = std::make_pair(dev, code);
    auto it = g_cache.find(key);
    if (it != g_cache.end()) {
        *out = it->second;
        return CHXQ_OK;
    }
    Nvrtc& n = nvrtc();
    if (!n.ok) return set_error(CHXQ_ERR_JIT, "ElementWiseNvrtc: %s", n.why.c_str());
    Driver& d = driver();
    if (!d.ok) return set_error(CHXQ_ERR_JIT, "ElementWiseNvrtc: %s", d.why.c_str());

    const std::string name = "fusion" + std::to_string(fusion_id);
    nvrtcProgram prog;
    int r = n.CreateProgram(&prog, code.c_str(), (name + ".cu").c_str(), 0, nullptr, nullptr);
    if (r != 0) return set_error(CHXQ_ERR_JIT, "nvrtcCreateProgram: %s", n.GetErrorString(r));
    const char* opts[] = {"--gpu-architecture=sm_100a", "--std=c++17", "-I/usr/local/cuda/include"};
    r = n.CompileProgram(prog, 3, opts);
    if (r != 0) {
        size_t ls = 0;
        n.GetProgramLogSize(prog, &ls);
        std::string log(ls + 1, '\0');
        if (ls) n.GetProgramLog(prog, &log[0]);
        n.DestroyProgram(&prog);
        return set_error(CHXQ_ERR_JIT, "NVRTC failed to compile %s: %s\n%.700s", name.c_str(), n.GetErrorString(r), log.c_str());
    }
    size_t sz = 0;
    n.GetCUBINSize(prog, &sz);
    std::vector<char> cubin(sz);
    r = n.GetCUBIN(prog, cubin.data());
    n.DestroyProgram(&prog);
    if (r != 0 || sz == 0) return set_error(CHXQ_ERR_JIT, "nvrtcGetCUBIN failed for %s", name.c_str());

    CUmodule mod;
    CUresult cr = d.ModuleLoadData(&mod, cubin.data());
    if (cr != CUDA_SUCCESS) return set_error(CHXQ_ERR_CUDA, "cuModuleLoadData failed with %d for %s", (int)cr, name.c_str());
    Loaded l{};
    cr = d.ModuleGetFunction(&l.vec, mod, name.c_str());
    if (cr != CUDA_SUCCESS) return set_error(CHXQ_ERR_CUDA, "kernel %s not found in the generated module (%d)", name.c_str(), (int)cr);
    cr = d.ModuleGetFunction(&l.scalar, mod, (name + "_s").c_str());
    if (cr != CUDA_SUCCESS) return set_error(CHXQ_ERR_CUDA, "kernel %s_s not found in the generated module (%d)", name.c_str(), (int)cr);
    g_cache.emplace(key, l);
    *out = l;
    return CHXQ_OK;
}

}  // namespace
}  // namespace chxq

using namespace chxq;

extern "C" int chxq_eltwise_codegen(
        const chxq_ew_node* nodes, int32_t n_nodes, const int32_t* input_ids, int32_t n_inputs, const int32_t* output_ids, int32_t n_outputs,
        const char* const* value_names, int32_t n_values, int32_t dtype, int32_t fusion_id, char* buf, size_t buf_len, size_t* needed) {
    CHXQ_CHECK_ARG(nodes && n_nodes > 0 && input_ids && n_inputs > 0 && output_ids && n_outputs > 0 && value_names && n_values > 0,
                   "eltwise codegen: empty group");
    CHXQ_CHECK_ARG(dtype == CHXQ_FLOAT16 || dtype == CHXQ_FLOAT32 || dtype == CHXQ_FLOAT64, "eltwise codegen: dtype %d is not a float type", dtype);
    auto valid = [&](int v) { return v >= 0 && v < n_values; };
    std::vector<int> producer(n_values, -1);
    for (int i = 0; i < n_nodes; ++i) {
        const chxq_ew_node& nd = nodes[i];
        CHXQ_CHECK_ARG(nd.op >= CHXQ_EW_IDENTITY && nd.op <= CHXQ_EW_CONSTANT, "eltwise codegen: cannot build a kernel for op code %d", nd.op);
        CHXQ_CHECK_ARG(valid(nd.output), "eltwise codegen: node %d has a bad output id", i);
        CHXQ_CHECK_ARG(producer[nd.output] < 0, "eltwise codegen: value %d is produced twice", nd.output);
        producer[nd.output] = i;
        for (int k = 0; k < n_operands(nd.op); ++k) CHXQ_CHECK_ARG(valid(nd.inputs[k]), "eltwise codegen: node %d has a bad input id", i);
    }
    std::set<int> is_input;
    for (int i = 0; i < n_inputs; ++i) {
        CHXQ_CHECK_ARG(valid(input_ids[i]) && producer[input_ids[i]] < 0, "eltwise codegen: bad group input %d", input_ids[i]);
        is_input.insert(input_ids[i]);
    }
    for (int i = 0; i < n_outputs; ++i) CHXQ_CHECK_ARG(valid(output_ids[i]) && producer[output_ids[i]] >= 0, "eltwise codegen: bad group output");

    auto vname = [&](int v) { return cleanse(value_names[v], "v_"); };
    const bool is_half = dtype == CHXQ_FLOAT16;
    const char* store_t = dtype == CHXQ_FLOAT64 ? "double" : (is_half ? "__half" : "float");
    const char* comp_t = dtype == CHXQ_FLOAT64 ? "double" : "float";
    const int vec = dtype == CHXQ_FLOAT64 ? 2 : (is_half ? 8 : 4);

    std::ostringstream ce;
    ce << "// fused elementwise group " << fusion_id << ": " << n_nodes << " nodes, " << n_inputs << " inputs, " << n_outputs << " outputs\n";
    if (is_half) ce << "#include <cuda_fp16.h>\n";
    ce << "typedef " << store_t << " S;  // storage type\n";
    ce << "typedef " << comp_t << " T;  // arithmetic type\n";
    ce << "#define CHXQ_VEC " << vec << "\n";
    ce << "union Pack { uint4 u; S e[CHXQ_VEC]; };\n";
    if (is_half) {
        ce << "__device__ __forceinline__ T ld(S v) { return __half2float(v); }\n";
        ce << "__device__ __forceinline__ S st(T v) { return __float2half_rn(v); }\n";
    } else {
        ce << "__device__ __forceinline__ T ld(S v) { return v; }\n";
        ce << "__device__ __forceinline__ S st(T v) { return v; }\n";
    }
    bool has_sigmoid = false;
    for (int i = 0; i < n_nodes; ++i) has_sigmoid |= nodes[i].op == CHXQ_EW_SIGMOID;
    if (has_sigmoid) {
        ce << "__device__ __forceinline__ T sigmoid(T x) {\n";
        ce << "    const T one = 1;\n";
        ce << "    return one / (one + exp(-x));\n";
        ce << "}\n";
    }

    // Per-element body, nodes emitted in dependency order (Kahn, starting from the inputs and constants).
    ce << "__device__ __forceinline__ void fusion" << fusion_id << "_elem(";
    for (int i = 0; i < n_inputs; ++i) ce << (i ? ", " : "") << "const T " << vname(input_ids[i]);
    for (int i = 0; i < n_outputs; ++i) ce << ", T& " << cleanse(value_names[output_ids[i]], "r_");
    ce << ") {\n";
    std::vector<int> pending(n_nodes);
    std::vector<std::vector<int>> users(n_values);
    std::queue<int> q;
    for (int i = 0; i < n_nodes; ++i) {
        pending[i] = n_operands(nodes[i].op);
        for (int k = 0; k < pending[i]; ++k) users[nodes[i].inputs[k]].push_back(i);
    }
    for (int i = 0; i < n_inputs; ++i) q.push(input_ids[i]);
    char num[64];
    for (int i = 0; i < n_nodes; ++i) {
        if (nodes[i].op != CHXQ_EW_CONSTANT) continue;
        snprintf(num, sizeof(num), dtype == CHXQ_FLOAT64 ? "%.17g" : "%.9g", nodes[i].constant);
        std::string lit = num;
        if (lit.find_first_of(".eEni") == std::string::npos) lit += ".0";
        ce << "    const T " << vname(nodes[i].output) << " = (T)(" << lit << ");  // Constant\n";
        q.push(nodes[i].output);
    }
    int emitted = 0;
    while (!q.empty()) {
        const int v = q.front();
        q.pop();
        for (int ni : users[v]) {
            if (--pending[ni] != 0) continue;
            const chxq_ew_node& nd = nodes[ni];
            std::string a = vname(nd.inputs[0]);
            std::string rhs;
            switch (nd.op) {
                case CHXQ_EW_IDENTITY: rhs = a; break;
                case CHXQ_EW_TANH: rhs = "tanh(" + a + ")"; break;
                case CHXQ_EW_EXP: rhs = "exp(" + a + ")"; break;
                case CHXQ_EW_SIGMOID: rhs = "sigmoid(" + a + ")"; break;
                case CHXQ_EW_ADD: rhs = a + " + " + vname(nd.inputs[1]); break;
                case CHXQ_EW_SUB: rhs = a + " - " + vname(nd.inputs[1]); break;
                case CHXQ_EW_MUL: rhs = a + " * " + vname(nd.inputs[1]); break;
                case CHXQ_EW_DIV: rhs = a + " / " + vname(nd.inputs[1]); break;
            }
            ce << "    const T " << vname(nd.output) << " = " << rhs << ";  // " << op_comment(nd.op) << "\n";
            ++emitted;
            q.push(nd.output);
        }
    }
    int n_const = 0;
    for (int i = 0; i < n_nodes; ++i) n_const += nodes[i].op == CHXQ_EW_CONSTANT;
    CHXQ_CHECK_ARG(emitted + n_const == n_nodes, "eltwise codegen: the group is cyclic or reads a value that is neither an input nor produced in it");
    for (int i = 0; i < n_outputs; ++i) ce << "    " << cleanse(value_names[output_ids[i]], "r_") << " = " << vname(output_ids[i]) << ";  // output\n";
    ce << "}\n";

    auto params = [&]() {
        std::ostringstream p;
        p << "size_t n";
        for (int i = 0; i < n_inputs; ++i) p << ", const S* __restrict__ " << cleanse(value_names[input_ids[i]], "i_");
        for (int i = 0; i < n_outputs; ++i) p << ", S* __restrict__ " << cleanse(value_names[output_ids[i]], "o_");
        return p.str();
    };
    auto scalar_body = [&](const char* idx) {
        std::ostringstream b;
        for (int i = 0; i < n_outputs; ++i) b << "        T " << cleanse(value_names[output_ids[i]], "r_") << ";\n";
        b << "        fusion" << fusion_id << "_elem(";
        for (int i = 0; i < n_inputs; ++i) b << (i ? ", " : "") << "ld(" << cleanse(value_names[input_ids[i]], "i_") << "[" << idx << "])";
        for (int i = 0; i < n_outputs; ++i) b << ", " << cleanse(value_names[output_ids[i]], "r_");
        b << ");\n";
        for (int i = 0; i < n_outputs; ++i)
            b << "        " << cleanse(value_names[output_ids[i]], "o_") << "[" << idx << "] = st(" << cleanse(value_names[output_ids[i]], "r_") << ");\n";
        return b.str();
    };

    // 128-bit vectorised kernel (all buffers 16-byte aligned) with a scalar tail.
    ce << "extern \"C\" __global__ void __launch_bounds__(256) fusion" << fusion_id << "(" << params() << ") {\n";
    ce << "    const size_t nv = n / CHXQ_VEC;\n";
    ce << "    const size_t stride = (size_t)gridDim.x * blockDim.x;\n";
    ce << "    const size_t t0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;\n";
    ce << "    for (size_t v = t0; v < nv; v += stride) {\n";
    for (int i = 0; i < n_inputs; ++i) {
        const std::string nm = cleanse(value_names[input_ids[i]], "i_");
        ce << "        Pack p" << nm << "; p" << nm << ".u = __ldcs(reinterpret_cast<const uint4*>(" << nm << ") + v);\n";
    }
    for (int i = 0; i < n_outputs; ++i) ce << "        Pack q" << cleanse(value_names[output_ids[i]], "o_") << ";\n";
    ce << "#pragma unroll\n";
    ce << "        for (int j = 0; j < CHXQ_VEC; ++j) {\n";
    for (int i = 0; i < n_outputs; ++i) ce << "            T " << cleanse(value_names[output_ids[i]], "r_") << ";\n";
    ce << "            fusion" << fusion_id << "_elem(";
    for (int i = 0; i < n_inputs; ++i) ce << (i ? ", " : "") << "ld(p" << cleanse(value_names[input_ids[i]], "i_") << ".e[j])";
    for (int i = 0; i < n_outputs; ++i) ce << ", " << cleanse(value_names[output_ids[i]], "r_");
    ce << ");\n";
    for (int i = 0; i < n_outputs; ++i)
        ce << "            q" << cleanse(value_names[output_ids[i]], "o_") << ".e[j] = st(" << cleanse(value_names[output_ids[i]], "r_") << ");\n";
    ce << "        }\n";
    for (int i = 0; i < n_outputs; ++i) {
        const std::string nm = cleanse(value_names[output_ids[i]], "o_");
        ce << "        __stcs(reinterpret_cast<uint4*>(" << nm << ") + v, q" << nm << ".u);\n";
    }
    ce << "    }\n";
    ce << "    for (size_t i = nv * CHXQ_VEC + t0; i < n; i += stride) {\n" << scalar_body("i") << "    }\n";
    ce << "}\n";
    // Scalar kernel for unaligned buffers.
    ce << "extern \"C\" __global__ void __launch_bounds__(256) fusion" << fusion_id << "_s(" << params() << ") {\n";
    ce << "    const size_t stride = (size_t)gridDim.x * blockDim.x;\n";
    ce << "    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {\n" << scalar_body("i") << "    }\n";
    ce << "}\n";

    const std::string text = ce.str();
    if (needed) *needed = text.size() + 1;
    if (buf == nullptr || buf_len < text.size() + 1) {
        if (buf != nullptr && buf_len > 0) buf[0] = '\0';
        return buf == nullptr ? CHXQ_OK : set_error(CHXQ_ERR_INVALID_ARGUMENT, "eltwise codegen: buffer of %zu bytes is too small (%zu needed)", buf_len, text.size() + 1);
    }
    memcpy(buf, text.c_str(), text.size() + 1);
    return CHXQ_OK;
}

extern "C" int chxq_eltwise_run(
        const char* code, int32_t fusion_id, const void* const* inputs, int32_t n_inputs, void* const* outputs, int32_t n_outputs, int64_t n,
        int32_t dtype, void* stream) {
    CHXQ_CHECK_ARG(code && code[0], "ElementWiseNvrtc: empty code");
    CHXQ_CHECK_ARG(inputs && n_inputs > 0, "ElementWiseNvrtc: no inputs");  // runtime/ops/nvrtc.cc:93 CHECK(!inputs.empty())
    CHXQ_CHECK_ARG(outputs && n_outputs > 0, "ElementWiseNvrtc: no outputs");
    CHXQ_CHECK_ARG(dtype == CHXQ_FLOAT16 || dtype == CHXQ_FLOAT32 || dtype == CHXQ_FLOAT64, "ElementWiseNvrtc: dtype %d is not a float type", dtype);
    CHXQ_CHECK_ARG(n >= 0 && n < (1ll << 31), "ElementWiseNvrtc: element count must be below 2^31");  // runtime/ops/nvrtc.cc:129
    if (n == 0) return CHXQ_OK;
    Loaded fn;
    int rc = compile_and_load(code, fusion_id, &fn);
    if (rc != CHXQ_OK) return rc;
    bool aligned = true;
    std::vector<const void*> in_ptrs(inputs, inputs + n_inputs);
    std::vector<void*> out_ptrs(outputs, outputs + n_outputs);
    for (const void* p : in_ptrs) {
        CHXQ_CHECK_ARG(p != nullptr, "ElementWiseNvrtc: null input buffer");
        aligned = aligned && (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
    }
    for (void* p : out_ptrs) {
        CHXQ_CHECK_ARG(p != nullptr, "ElementWiseNvrtc: null output buffer");
        aligned = aligned && (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
    }
    size_t nn = (size_t)n;
    std::vector<void*> args;
    args.push_back(&nn);
    for (auto& p : in_ptrs) args.push_back(&p);
    for (auto& p : out_ptrs) args.push_back(&p);
    const int vec = dtype == CHXQ_FLOAT64 ? 2 : (dtype == CHXQ_FLOAT16 ? 8 : 4);
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t work = aligned ? (n + vec - 1) / vec : n;
    int64_t blocks = (work + 255) / 256;
    if (blocks > (int64_t)sms * 32) blocks = (int64_t)sms * 32;
    if (blocks < 1) blocks = 1;
    CUresult cr = driver().LaunchKernel(aligned ? fn.vec : fn.scalar, (unsigned)blocks, 1, 1, 256, 1, 1, 0, reinterpret_cast<CUstream>(stream),
                                        args.data(), nullptr);
    if (cr != CUDA_SUCCESS) return set_error(CHXQ_ERR_CUDA, "cuLaunchKernel(fusion%d) failed with %d", fusion_id, (int)cr);
    count_launch(1);
    return CHXQ_OK;
}
