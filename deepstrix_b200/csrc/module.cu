// Code-object verbs of the device FFI: load a cubin / fatbin image from memory, look kernels up by
// name, launch them with the CUDA "kernelParams" ABI, and the stream memory operations.
//
// Reference counterparts (paths relative to the deepstrix repository):
//   crates/v4flash-hip/src/module.rs:28-57     Module::load_data, get_function with its name -> handle cache
//   crates/v4flash-hip/src/module.rs:141-171   Function::launch_raw(cfg, stream, void** args)
//   crates/v4flash-hip/src/launch.rs:25-40     LaunchConfig {grid, block, shared_mem_bytes}
//   crates/v4flash-hip/src/sys.rs:290-302      hipStreamWaitValue32 / hipStreamWriteValue32
//   crates/v4flash-hip/src/sys.rs:317-330      hipModuleLoadData / Unload / GetFunction / LaunchKernel
//   crates/v4flash-kernels/build.rs:114-119    kernels embedded as code-object blobs (include_bytes!)
// These are driver-API calls (cuModule*, cuLaunchKernel, cuStream*Value32); the library links only the
// runtime, so the entry points are looked up through cudaGetDriverEntryPoint.  The runtime's primary
// context of the current device is the context they act on.
#include <cuda.h>

#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "dsx_common.cuh"

namespace dsx {
namespace {

template <typename Fn>
int driver_fn(const char* name, Fn* out) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    DSX_CUDA(cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &qres));
    if (qres != cudaDriverEntryPointSuccess || !p) return set_error(DSX_ERR_UNSUPPORTED, "the driver has no %s", name);
    *out = reinterpret_cast<Fn>(p);
    return DSX_OK;
}

int driver_error(CUresult r, const char* what) {
    typedef CUresult (*GetErrorStringFn)(CUresult, const char**);
    static GetErrorStringFn get_str = nullptr;
    const char* msg = nullptr;
    if (!get_str) driver_fn("cuGetErrorString", &get_str);
    if (get_str) get_str(r, &msg);
    return set_error((int)r, "%s failed: %s (CUresult %d)", what, msg ? msg : "unknown error", (int)r);
}

#define DSX_DRV(call, what)                                  \
    do {                                                     \
        const CUresult _r = (call);                          \
        if (_r != CUDA_SUCCESS) return driver_error(_r, what); \
    } while (0)

}  // namespace
}  // namespace dsx

using namespace dsx;

struct dsx_module {
    CUmodule raw = nullptr;
    int device = 0;                           // current at load; unload runs under it
    std::mutex mu;
    std::map<std::string, CUfunction> functions;   // cuModuleGetFunction results by name
};

extern "C" {

int dsx_module_load_data(const void* image, dsx_module** module) {
    DSX_REQUIRE(image && module, "module_load_data: null argument");
    typedef CUresult (*LoadDataFn)(CUmodule*, const void*);
    static LoadDataFn load = nullptr;
    if (!load)
        if (int rc = driver_fn("cuModuleLoadData", &load)) return rc;
    DSX_CUDA(cudaFree(nullptr));   // makes the runtime's primary context current on this thread
    dsx_module* m = new (std::nothrow) dsx_module();
    if (!m) return set_error(DSX_ERR_NOMEM, "module_load_data: out of host memory");
    cudaGetDevice(&m->device);
    const CUresult r = load(&m->raw, image);
    if (r != CUDA_SUCCESS) {
        delete m;
        return driver_error(r, "cuModuleLoadData");
    }
    *module = m;
    return DSX_OK;
}

int dsx_module_unload(dsx_module* m) {
    if (!m) return DSX_OK;
    typedef CUresult (*UnloadFn)(CUmodule);
    static UnloadFn unload = nullptr;
    if (!unload)
        if (int rc = driver_fn("cuModuleUnload", &unload)) return rc;
    int prev = 0;
    cudaGetDevice(&prev);
    if (prev != m->device) cudaSetDevice(m->device);
    const CUresult r = unload(m->raw);
    if (prev != m->device) cudaSetDevice(prev);
    delete m;
    if (r != CUDA_SUCCESS) return driver_error(r, "cuModuleUnload");
    return DSX_OK;
}

int dsx_module_get_function(dsx_module* m, const char* name, dsx_function_t* fn) {
    DSX_REQUIRE(m && name && fn, "module_get_function: null argument");
    typedef CUresult (*GetFunctionFn)(CUfunction*, CUmodule, const char*);
    static GetFunctionFn get = nullptr;
    if (!get)
        if (int rc = driver_fn("cuModuleGetFunction", &get)) return rc;
    std::lock_guard<std::mutex> lock(m->mu);
    auto it = m->functions.find(name);
    if (it == m->functions.end()) {
        CUfunction f = nullptr;
        const CUresult r = get(&f, m->raw, name);
        if (r != CUDA_SUCCESS) return driver_error(r, "cuModuleGetFunction");
        it = m->functions.emplace(name, f).first;
    }
    *fn = it->second;
    return DSX_OK;
}

int dsx_function_set_max_shared(dsx_function_t fn, uint32_t bytes) {
    DSX_REQUIRE(fn, "function_set_max_shared: null function");
    typedef CUresult (*SetAttrFn)(CUfunction, CUfunction_attribute, int);
    static SetAttrFn set_attr = nullptr;
    if (!set_attr)
        if (int rc = driver_fn("cuFuncSetAttribute", &set_attr)) return rc;
    DSX_DRV(set_attr((CUfunction)fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, (int)bytes), "cuFuncSetAttribute");
    return DSX_OK;
}

int dsx_function_launch(dsx_function_t fn, const uint32_t grid[3], const uint32_t block[3], uint32_t shared_bytes, dsx_stream_t stream,
                        void** params) {
    DSX_REQUIRE(fn && grid && block, "function_launch: null argument");
    typedef CUresult (*LaunchFn)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream, void**, void**);
    static LaunchFn launch = nullptr;
    if (!launch)
        if (int rc = driver_fn("cuLaunchKernel", &launch)) return rc;
    count_launch();
    DSX_DRV(launch((CUfunction)fn, grid[0], grid[1], grid[2], block[0], block[1], block[2], shared_bytes, (CUstream)stream, params, nullptr),
            "cuLaunchKernel");
    return DSX_OK;
}

// ---- executable graphs whose kernel nodes can be re-pointed (crates/v4flash-hip/src/sys.rs:360-382:
// hipGraphGetNodes, hipGraphKernelNodeGetParams, hipGraphExecKernelNodeSetParams; src/graph.rs)
int dsx_graph_end_capture_keep(dsx_stream_t stream, dsx_graph_t* graph_exec, void** graph) {
    DSX_REQUIRE(graph_exec && graph, "graph_end_capture_keep: null argument");
    cudaGraph_t g = nullptr;
    DSX_CUDA(cudaStreamEndCapture((cudaStream_t)stream, &g));
    cudaGraphExec_t ge = nullptr;
    const cudaError_t e = cudaGraphInstantiate(&ge, g, 0);
    if (e != cudaSuccess) {
        cudaGraphDestroy(g);
        DSX_CUDA(e);
    }
    *graph_exec = ge;
    *graph = g;
    return DSX_OK;
}

int dsx_graph_template_destroy(void* graph) {
    if (graph) DSX_CUDA(cudaGraphDestroy((cudaGraph_t)graph));
    return DSX_OK;
}

int dsx_graph_kernel_nodes(void* graph, void** nodes, size_t* count) {
    DSX_REQUIRE(graph && count, "graph_kernel_nodes: null argument");
    size_t n = 0;
    DSX_CUDA(cudaGraphGetNodes((cudaGraph_t)graph, nullptr, &n));
    std::vector<cudaGraphNode_t> all(n);
    if (n) DSX_CUDA(cudaGraphGetNodes((cudaGraph_t)graph, all.data(), &n));
    size_t k = 0;
    for (size_t i = 0; i < n; i++) {
        cudaGraphNodeType ty;
        DSX_CUDA(cudaGraphNodeGetType(all[i], &ty));
        if (ty != cudaGraphNodeTypeKernel) continue;
        if (nodes && k < *count) nodes[k] = all[i];
        k++;
    }
    *count = k;   // kernel nodes in the graph (nodes[] received min(capacity, k) of them)
    return DSX_OK;
}

int dsx_graph_exec_kernel_node_set_params(dsx_graph_t graph_exec, void* node, dsx_function_t fn, const uint32_t grid[3],
                                          const uint32_t block[3], uint32_t shared_bytes, void** params) {
    DSX_REQUIRE(graph_exec && node && params, "graph_exec_kernel_node_set_params: null argument");
    typedef CUresult (*GetFn)(CUgraphNode, CUDA_KERNEL_NODE_PARAMS*);
    typedef CUresult (*SetFn)(CUgraphExec, CUgraphNode, const CUDA_KERNEL_NODE_PARAMS*);
    static GetFn get = nullptr;
    static SetFn set = nullptr;
    if (!get)
        if (int rc = driver_fn("cuGraphKernelNodeGetParams", &get)) return rc;
    if (!set)
        if (int rc = driver_fn("cuGraphExecKernelNodeSetParams", &set)) return rc;
    CUDA_KERNEL_NODE_PARAMS p;
    DSX_DRV(get((CUgraphNode)node, &p), "cuGraphKernelNodeGetParams");
    if (fn) p.func = (CUfunction)fn;   // null: keep the node's kernel
    if (grid) { p.gridDimX = grid[0]; p.gridDimY = grid[1]; p.gridDimZ = grid[2]; }
    if (block) { p.blockDimX = block[0]; p.blockDimY = block[1]; p.blockDimZ = block[2]; p.sharedMemBytes = shared_bytes; }
    p.kernelParams = params;
    p.extra = nullptr;
    DSX_DRV(set((CUgraphExec)graph_exec, (CUgraphNode)node, &p), "cuGraphExecKernelNodeSetParams");
    return DSX_OK;
}

int dsx_stream_wait_value32(dsx_stream_t stream, void* dptr, uint32_t value, uint32_t flags) {
    DSX_REQUIRE(dptr && flags <= 3, "stream_wait_value32: null address or flags %u (0 = >=, 1 = ==, 2 = and, 3 = nor)", flags);
    typedef CUresult (*WaitFn)(CUstream, CUdeviceptr, cuuint32_t, unsigned);
    static WaitFn wait = nullptr;
    if (!wait)
        if (int rc = driver_fn("cuStreamWaitValue32", &wait)) return rc;
    static const unsigned kFlag[4] = {CU_STREAM_WAIT_VALUE_GEQ, CU_STREAM_WAIT_VALUE_EQ, CU_STREAM_WAIT_VALUE_AND, CU_STREAM_WAIT_VALUE_NOR};
    DSX_DRV(wait((CUstream)stream, (CUdeviceptr)dptr, value, kFlag[flags]), "cuStreamWaitValue32");
    return DSX_OK;
}

int dsx_stream_write_value32(dsx_stream_t stream, void* dptr, uint32_t value) {
    DSX_REQUIRE(dptr, "stream_write_value32: null address");
    typedef CUresult (*WriteFn)(CUstream, CUdeviceptr, cuuint32_t, unsigned);
    static WriteFn write = nullptr;
    if (!write)
        if (int rc = driver_fn("cuStreamWriteValue32", &write)) return rc;
    DSX_DRV(write((CUstream)stream, (CUdeviceptr)dptr, value, CU_STREAM_WRITE_VALUE_DEFAULT), "cuStreamWriteValue32");
    return DSX_OK;
}

}  // extern "C"
