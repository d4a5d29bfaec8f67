/*
 * vxb200_provider.c - the B200 W8A8 route as a VolvoxAI backend provider.
 *
 * Built against the reference's own public header (native/include/volvoxai_backend.h, found
 * through -I at build time; nothing of it is copied here) and linked against libvxb200.so.
 * It fills one VxBackendProvider descriptor (volvoxai_backend.h:168-259) and hands it to
 * vx_backend_register_provider (:269-271), following the template of
 * examples/backend_sdk/host_backend.c: whole-graph compile -> context_create ->
 * context_execute(HOST-borrowed inputs, VxBackendOutputSink copies the outputs).
 *
 *   compile          opens the package named by VxModelSource (graph.json + SafeTensors) with
 *                    vxb_package_open; a graph with any operator this route does not serve is
 *                    BACKEND_UNSUPPORTED, so the host's policy moves on to its next candidate;
 *                    the logical input/output specs must equal the package's; graphs with
 *                    PackedLinear are attested for DYNAMIC_I8 arithmetic only
 *   context_create   one VxbContext + one compiled program per context (contexts never share
 *                    mutable scratch, docs/backend-sdk.md:75-95)
 *   context_execute  validates the complete binding set, one device-resident forward pass,
 *                    every declared output written exactly once through the sink
 *
 * Name "b200-w8a8".  The device is VOLVOXAI_CUDA_DEVICE (the reference's selector), default 0; a
 * machine without an sm_100a device reports BACKEND_UNAVAILABLE at runtime_create, which omits
 * the provider from that runtime.
 */
#include "volvoxai_backend.h"

#include "../../include/vxb200_package.h"

#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define VXB_PROVIDER_NAME "b200-w8a8"

typedef struct { int device; } ProviderRuntime;
typedef struct { ProviderRuntime* runtime; VxbPackage* package; int has_packed_linear; } ProviderCompiled;
typedef struct { ProviderCompiled* compiled; VxbContext* ctx; VxbProgram* program; int closed; } ProviderContext;

static void fill_report(VxReport* report, VxStatus status, VxStage stage, VxOperationCode code, const char* message) {
    if (!report || report->struct_size != sizeof(*report)) return;
    memset(report, 0, sizeof(*report));
    report->struct_size = sizeof(*report);
    report->status = status; report->stage = stage; report->code = code;
    snprintf(report->backend, sizeof(report->backend), "%s", VXB_PROVIDER_NAME);
    snprintf(report->device, sizeof(report->device), "%s", "cuda:sm_100a");
    snprintf(report->message, sizeof(report->message), "%s", message ? message : "");
}

static int policy_names_us(const VxBackendPolicy* policy) {
    if (!policy || policy->struct_size != sizeof(*policy) || !policy->backends) return 0;
    for (size_t i = 0; i < policy->backend_count; i++)
        if (policy->backends[i] && !strcmp(policy->backends[i], VXB_PROVIDER_NAME)) return 1;
    return 0;
}

static VxDataType to_vx_dtype(uint32_t dt) { return (VxDataType)dt; }   /* the numeric values are the reference's */

/* A logical spec equals a package tensor: same name, dtype, rank, fixed host dimensions. */
static int spec_matches(const VxTensorSpec* spec, const VxbPackage* package, int is_output, uint32_t index) {
    if (!spec || spec->struct_size != sizeof(*spec) || !spec->name || spec->location != VX_MEMORY_HOST) return 0;
    if (strcmp(spec->name, vxb_package_io_name(package, is_output, index)) ||
        spec->dtype != to_vx_dtype(vxb_package_io_dtype(package, is_output, index)) ||
        spec->rank != vxb_package_io_rank(package, is_output, index)) return 0;
    for (uint32_t a = 0; a < spec->rank; a++) {
        const VxDimensionConstraint* d = &spec->dimensions[a];
        const int64_t want = vxb_package_io_dim(package, is_output, index, a);
        if (d->struct_size != sizeof(*d) || d->kind != VX_DIMENSION_FIXED || d->symbol || d->min != want || d->max != want ||
            d->multiple_of != 1) return 0;
    }
    return 1;
}

static VxStatus provider_runtime_create(void* user_data, const VxRuntimeOptions* options, void** out_runtime, VxReport* report) {
    (void)user_data;
    if (!out_runtime) return VX_STATUS_INVALID_ARGUMENT;
    *out_runtime = NULL;
    if (!options || options->struct_size != sizeof(*options)) return VX_STATUS_INVALID_ARGUMENT;
    int device = 0;
    const char* env = getenv("VOLVOXAI_CUDA_DEVICE");
    if (env) device = atoi(env);
    /* probe: a context can only be created on an sm_100a device */
    VxbContext* probe = NULL;
    if (vxb_context_create(device, NULL, &probe) != 1) {
        fill_report(report, VX_STATUS_BACKEND_UNAVAILABLE, VX_STAGE_RUNTIME_CREATE, VX_CODE_NONE, vxb_last_error());
        return VX_STATUS_BACKEND_UNAVAILABLE;
    }
    vxb_context_destroy(probe);
    ProviderRuntime* runtime = (ProviderRuntime*)calloc(1, sizeof(*runtime));
    if (!runtime) return VX_STATUS_OUT_OF_MEMORY;
    runtime->device = device;
    *out_runtime = runtime;
    fill_report(report, VX_STATUS_OK, VX_STAGE_RUNTIME_CREATE, VX_CODE_NONE, "b200-w8a8 provider runtime created");
    return VX_STATUS_OK;
}

static void provider_runtime_destroy(void* runtime) { free(runtime); }

static void provider_compiled_destroy(void* instance) {
    ProviderCompiled* compiled = (ProviderCompiled*)instance;
    if (!compiled) return;
    vxb_package_close(compiled->package);
    free(compiled);
}

static VxStatus provider_compile(void* runtime_instance, const VxBackendCompileInput* input, const VxBackendPolicy* policy,
                                 void** out_compiled, VxBackendShapeDomainAttestation* attestation, VxReport* report) {
    if (!runtime_instance || !input || input->struct_size != sizeof(*input) || !input->source ||
        input->source->struct_size != sizeof(*input->source) || !input->graph_fingerprint ||
        !input->shape_domain_proof_identity || !out_compiled || !attestation ||
        attestation->struct_size != sizeof(*attestation) || !policy_names_us(policy))
        return VX_STATUS_INVALID_ARGUMENT;
    *out_compiled = NULL;
    VxbPackage* package = NULL;
    if (vxb_package_open(input->source->graph_path, input->source->weight_paths, input->source->weight_path_count, &package) != 1) {
        fill_report(report, VX_STATUS_BACKEND_UNSUPPORTED, VX_STAGE_COMPILE, VX_CODE_BACKEND_UNSUPPORTED, vxb_last_error());
        return VX_STATUS_BACKEND_UNSUPPORTED;
    }
    int ok = input->input_count == vxb_package_io_count(package, 0) && input->output_count == vxb_package_io_count(package, 1) &&
             input->inputs && input->outputs;
    for (uint32_t i = 0; ok && i < input->input_count; i++) ok = spec_matches(&input->inputs[i], package, 0, i);
    for (uint32_t i = 0; ok && i < input->output_count; i++) ok = spec_matches(&input->outputs[i], package, 1, i);
    if (!ok) {
        vxb_package_close(package);
        fill_report(report, VX_STATUS_INVALID_ARGUMENT, VX_STAGE_COMPILE, VX_CODE_NONE,
                    "logical input/output specifications differ from the package's graph");
        return VX_STATUS_INVALID_ARGUMENT;
    }
    int has_packed = 0;
    uint64_t largest = 0, resident = 0;
    for (uint32_t i = 0; i < vxb_package_node_count(package); i++)
        if (!strcmp(vxb_package_node_op(package, i), "PackedLinear")) has_packed = 1;
    for (int side = 0; side < 2; side++)
        for (uint32_t i = 0; i < vxb_package_io_count(package, side); i++) {
            const uint64_t b = vxb_package_io_bytes(package, side, i);
            largest = b > largest ? b : largest; resident += b;
        }
    /* this route computes PackedLinear with dynamic per-row int8 activations: it cannot attest another arithmetic */
    if (has_packed && input->packed_arithmetic != VX_PACKED_ARITHMETIC_DYNAMIC_I8) {
        vxb_package_close(package);
        fill_report(report, VX_STATUS_BACKEND_UNSUPPORTED, VX_STAGE_COMPILE, VX_CODE_BACKEND_UNSUPPORTED,
                    "PackedLinear is served with DYNAMIC_I8 arithmetic only");
        return VX_STATUS_BACKEND_UNSUPPORTED;
    }
    ProviderCompiled* compiled = (ProviderCompiled*)calloc(1, sizeof(*compiled));
    if (!compiled) { vxb_package_close(package); return VX_STATUS_OUT_OF_MEMORY; }
    compiled->runtime = (ProviderRuntime*)runtime_instance;
    compiled->package = package;
    compiled->has_packed_linear = has_packed;
    *out_compiled = compiled;
    attestation->graph_fingerprint = input->graph_fingerprint;
    attestation->shape_domain_proof_identity = input->shape_domain_proof_identity;
    attestation->maximum_tensor_bytes = largest;
    attestation->maximum_resident_bytes = resident;
    attestation->has_resource_limit = 0;
    attestation->packed_arithmetic = has_packed ? VX_PACKED_ARITHMETIC_DYNAMIC_I8 : VX_PACKED_ARITHMETIC_UNSPECIFIED;
    fill_report(report, VX_STATUS_OK, VX_STAGE_COMPILE, VX_CODE_NONE, "package compiled for the B200 W8A8 route");
    if (report && report->struct_size == sizeof(*report)) {
        report->route_attested = 1;
        report->operator_fallback_used = 0;
        snprintf(report->route_evidence, sizeof(report->route_evidence), "provider=%s;nodes=%u;route=sm100a-tcgen05-all",
                 VXB_PROVIDER_NAME, vxb_package_node_count(package));
        snprintf(report->fallback_evidence, sizeof(report->fallback_evidence), "%s", "operator=none");
    }
    return VX_STATUS_OK;
}

static void provider_context_destroy(void* instance) {
    ProviderContext* context = (ProviderContext*)instance;
    if (!context) return;
    vxb_program_destroy(context->program);
    vxb_context_destroy(context->ctx);
    free(context);
}

static VxStatus provider_context_create(void* compiled_instance, const VxContextOptions* options, void** out_context, VxReport* report) {
    if (!out_context) return VX_STATUS_INVALID_ARGUMENT;
    *out_context = NULL;
    ProviderCompiled* compiled = (ProviderCompiled*)compiled_instance;
    if (!compiled || !options || options->struct_size != sizeof(*options)) return VX_STATUS_INVALID_ARGUMENT;
    if (options->decode_row_mode != VX_DECODE_ROW_DISABLED) return VX_STATUS_BACKEND_UNSUPPORTED;
    ProviderContext* context = (ProviderContext*)calloc(1, sizeof(*context));
    if (!context) return VX_STATUS_OUT_OF_MEMORY;
    context->compiled = compiled;
    if (vxb_context_create(compiled->runtime->device, NULL, &context->ctx) != 1 ||
        vxb_program_compile(context->ctx, compiled->package, &context->program) != 1) {
        fill_report(report, VX_STATUS_OUT_OF_MEMORY, VX_STAGE_CONTEXT_CREATE, VX_CODE_NONE, vxb_last_error());
        provider_context_destroy(context);
        return VX_STATUS_OUT_OF_MEMORY;
    }
    *out_context = context;
    fill_report(report, VX_STATUS_OK, VX_STAGE_CONTEXT_CREATE, VX_CODE_NONE, "weights repacked on the device");
    return VX_STATUS_OK;
}

static VxStatus provider_context_execute(void* instance, const VxTensorBinding* inputs, size_t input_count,
                                         const VxBackendOutputSink* sink, VxReport* report) {
    enum { kMaxIo = 16 };
    ProviderContext* context = (ProviderContext*)instance;
    if (!context || context->closed || !inputs || !sink || sink->struct_size != sizeof(*sink) || !sink->write)
        return VX_STATUS_INVALID_ARGUMENT;
    const VxbPackage* package = context->compiled->package;
    const uint32_t n_in = vxb_package_io_count(package, 0), n_out = vxb_package_io_count(package, 1);
    if (input_count != n_in || n_in > kMaxIo || n_out > kMaxIo) return VX_STATUS_INVALID_ARGUMENT;
    /* validate the complete binding set before anything is dispatched: by name, each exactly once */
    const void* in_ptr[kMaxIo] = {0}; size_t in_bytes[kMaxIo] = {0};
    for (size_t b = 0; b < input_count; b++) {
        const VxTensorBinding* binding = &inputs[b];
        if (binding->struct_size != sizeof(*binding) || !binding->name || !binding->data || binding->location != VX_MEMORY_HOST)
            return VX_STATUS_INVALID_ARGUMENT;
        uint32_t slot = n_in;
        for (uint32_t i = 0; i < n_in; i++) if (!strcmp(binding->name, vxb_package_io_name(package, 0, i))) slot = i;
        if (slot == n_in || in_ptr[slot] || binding->dtype != to_vx_dtype(vxb_package_io_dtype(package, 0, slot)) ||
            binding->rank != vxb_package_io_rank(package, 0, slot) || binding->byte_size != vxb_package_io_bytes(package, 0, slot))
            return VX_STATUS_INVALID_ARGUMENT;
        for (uint32_t a = 0; a < binding->rank; a++)
            if (binding->shape[a] != vxb_package_io_dim(package, 0, slot, a)) return VX_STATUS_INVALID_ARGUMENT;
        in_ptr[slot] = binding->data; in_bytes[slot] = binding->byte_size;
    }
    void* out_ptr[kMaxIo] = {0}; size_t out_bytes[kMaxIo] = {0};
    VxStatus status = VX_STATUS_OK;
    for (uint32_t i = 0; i < n_out; i++) {
        out_bytes[i] = (size_t)vxb_package_io_bytes(package, 1, i);
        out_ptr[i] = malloc(out_bytes[i]);
        if (!out_ptr[i]) status = VX_STATUS_OUT_OF_MEMORY;
    }
    if (status == VX_STATUS_OK) {
        const int rc = vxb_program_execute(context->program, in_ptr, in_bytes, n_in, out_ptr, out_bytes, n_out);
        if (rc != 1) {
            status = rc == 0 ? VX_STATUS_INVALID_ARGUMENT : VX_STATUS_EXECUTION_FAILED;
            fill_report(report, status, VX_STAGE_EXECUTE, VX_CODE_NONE, vxb_last_error());
        }
    }
    for (uint32_t i = 0; status == VX_STATUS_OK && i < n_out; i++) {
        int64_t shape[VX_MAX_TENSOR_RANK] = {0};
        const uint32_t rank = vxb_package_io_rank(package, 1, i);
        for (uint32_t a = 0; a < rank; a++) shape[a] = vxb_package_io_dim(package, 1, i, a);
        status = sink->write(sink->user_data, vxb_package_io_name(package, 1, i), to_vx_dtype(vxb_package_io_dtype(package, 1, i)),
                             shape, rank, out_ptr[i], out_bytes[i]);
    }
    for (uint32_t i = 0; i < n_out; i++) free(out_ptr[i]);
    if (status != VX_STATUS_OK) return status;
    fill_report(report, VX_STATUS_OK, VX_STAGE_EXECUTE, VX_CODE_NONE, "forward pass executed on the device");
    if (report && report->struct_size == sizeof(*report)) {
        report->route_attested = 1;
        report->operator_fallback_used = 0;
        snprintf(report->route_evidence, sizeof(report->route_evidence), "provider=%s;%s", VXB_PROVIDER_NAME,
                 vxb_program_route_evidence(context->program));
    }
    return VX_STATUS_OK;
}

static VxStatus provider_context_close(void* instance, VxReport* report) {
    ProviderContext* context = (ProviderContext*)instance;
    (void)report;
    if (!context) return VX_STATUS_INVALID_ARGUMENT;
    context->closed = 1;
    return VX_STATUS_OK;
}

/* Fills *provider with this route's descriptor (for hosts that compose descriptors themselves). */
__attribute__((visibility("default"))) void vxb200_provider_descriptor(VxBackendProvider* provider) {
    const VxBackendProvider descriptor = {
        .struct_size = sizeof(VxBackendProvider),
        .abi_version = VX_BACKEND_ABI_VERSION,
        .name = VXB_PROVIDER_NAME,
        .shape_domain = {
            .struct_size = sizeof(VxBackendShapeDomainCapability),
            .proof_protocol = VX_BACKEND_SHAPE_PROOF_PROTOCOL,
            .resource_protocol = VX_BACKEND_RESOURCE_PROTOCOL,
            .support = VX_BACKEND_SHAPE_DOMAIN_FULL,   /* fixed shapes only: the whole (one-point) domain is attested or rejected */
        },
        .runtime_create = provider_runtime_create,
        .runtime_destroy = provider_runtime_destroy,
        .compile = provider_compile,
        .compiled_destroy = provider_compiled_destroy,
        .context_create = provider_context_create,
        .context_execute = provider_context_execute,
        .context_close = provider_context_close,
        .context_destroy = provider_context_destroy,
        .exact_contract_marker = VX_BACKEND_PROVIDER_EXACT_CONTRACT_MARKER,
        .exact_contract_extent = sizeof(VxBackendProvider),
    };
    *provider = descriptor;
}

/* Registers the provider with the host process (call before CreateRuntime). */
__attribute__((visibility("default"))) VxStatus vxb200_provider_register(VxReport* report) {
    VxBackendProvider provider;
    vxb200_provider_descriptor(&provider);
    return vx_backend_register_provider(&provider, report);
}
