/*
 * fake_host.c - a stand-in for the reference's runtime, for tests of the backend provider only
 * (test infrastructure; never part of the product).
 *
 * Compiled against the reference's public header where the reference checkout exists (recipe:
 * oracle/Makefile, output oracle/_ref/libvxfakehost.so).  It defines
 * vx_backend_register_provider with the reference's descriptor checks restated
 * (provider_descriptor_valid / provider_name_valid, native/src/runtime/backend_sdk.c:92-139),
 * keeps the registered descriptor, and drives it the way the runtime does - runtime_create,
 * compile, context_create, context_execute with HOST bindings and an output sink that copies
 * before write() returns - behind flat C entry points a ctypes test can call.
 */
#include "volvoxai_backend.h"

#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define API __attribute__((visibility("default")))

static VxBackendProvider g_provider;
static int g_registered;
static void* g_runtime; static void* g_compiled; static void* g_context;
static VxReport g_report;

static int name_valid(const char* name) {
    if (!name) return 0;
    const size_t length = strlen(name);
    if (!length || length >= VX_BACKEND_NAME_CAPACITY || name[0] < 'a' || name[0] > 'z') return 0;
    for (size_t i = 1; i < length; i++) {
        const unsigned char c = (unsigned char)name[i];
        if (!((c >= 'a' && c <= 'z') || (c >= '0' && c <= '9') || c == '.' || c == '_' || c == '-')) return 0;
    }
    /* built-in names are reserved */
    const char* reserved[] = {"cpu", "cuda", "vulkan", "opengl", "metal", "webgpu"};
    for (size_t i = 0; i < sizeof reserved / sizeof reserved[0]; i++) if (!strcmp(name, reserved[i])) return 0;
    return 1;
}

static int descriptor_valid(const VxBackendProvider* p) {
    const VxBackendShapeDomainCapability* c = p ? &p->shape_domain : NULL;
    return p && p->struct_size == sizeof(*p) && p->abi_version == VX_BACKEND_ABI_VERSION &&
        p->exact_contract_marker == VX_BACKEND_PROVIDER_EXACT_CONTRACT_MARKER && p->exact_contract_extent == sizeof(*p) &&
        name_valid(p->name) && p->flags == 0 &&
        c->struct_size == sizeof(*c) && c->proof_protocol && c->resource_protocol &&
        !strcmp(c->proof_protocol, VX_BACKEND_SHAPE_PROOF_PROTOCOL) && !strcmp(c->resource_protocol, VX_BACKEND_RESOURCE_PROTOCOL) &&
        (c->support == VX_BACKEND_SHAPE_DOMAIN_FULL || c->support == VX_BACKEND_SHAPE_DOMAIN_UNSUPPORTED) &&
        p->runtime_create && p->runtime_destroy && p->compile && p->compiled_destroy &&
        (!!p->compiled_batch_contract == !!p->context_execute_batch) && p->context_create && p->context_execute && p->context_destroy;
}

API VxStatus vx_backend_register_provider(const VxBackendProvider* provider, VxReport* report) {
    if (!report || report->struct_size != sizeof(*report)) return VX_STATUS_INVALID_ARGUMENT;
    if (!descriptor_valid(provider)) return VX_STATUS_INVALID_ARGUMENT;
    if (g_registered && !strcmp(g_provider.name, provider->name)) return VX_STATUS_INVALID_ARGUMENT;   /* duplicate name */
    g_provider = *provider;
    g_registered = 1;
    return VX_STATUS_OK;
}

static void fresh_report(void) {
    memset(&g_report, 0, sizeof g_report);
    g_report.struct_size = sizeof g_report;
}

API uint64_t fake_host_contract_marker(void) { return VX_BACKEND_PROVIDER_EXACT_CONTRACT_MARKER; }
API size_t fake_host_provider_struct_size(void) { return sizeof(VxBackendProvider); }
API const char* fake_host_message(void) { return g_report.message; }
API const char* fake_host_route_evidence(void) { return g_report.route_evidence; }
API int fake_host_route_attested(void) { return g_report.route_attested && !g_report.operator_fallback_used; }
API const char* fake_host_provider_name(void) { return g_registered ? g_provider.name : ""; }

/* Calls the provider library's registration function; returns its VxStatus. */
API int fake_host_register(VxStatus (*register_fn)(VxReport*)) {
    fresh_report();
    return (int)register_fn(&g_report);
}

/* Hands a deliberately wrong descriptor to the registration check: variant 0 = wrong struct size,
 * 1 = wrong contract marker, 2 = reserved name, 3 = missing required callback. Returns the status. */
API int fake_host_register_broken(void (*descriptor_fn)(VxBackendProvider*), int variant) {
    VxBackendProvider p;
    descriptor_fn(&p);
    if (variant == 0) p.struct_size -= 8;
    if (variant == 1) p.exact_contract_marker ^= 1;
    if (variant == 2) p.name = "cuda";
    if (variant == 3) p.context_execute = NULL;
    const int saved = g_registered;
    g_registered = 0;
    fresh_report();
    const int status = (int)vx_backend_register_provider(&p, &g_report);
    g_registered = saved;
    return status;
}

API int fake_host_runtime_create(void) {
    VxRuntimeOptions options = VX_RUNTIME_OPTIONS_INIT;
    fresh_report();
    return (int)g_provider.runtime_create(g_provider.user_data, &options, &g_runtime, &g_report);
}

/* names / dtypes / ranks / dims describe the logical inputs then the logical outputs (fixed shapes). */
API int fake_host_compile(const char* graph_path, const char* const* weight_paths, size_t weight_count,
                          const char* const* names, const uint32_t* dtypes, const uint32_t* ranks, const int64_t* dims,
                          size_t input_count, size_t output_count, int packed_arithmetic, const char* policy_name) {
    VxTensorSpec specs[32];
    if (input_count + output_count > 32) return (int)VX_STATUS_INVALID_ARGUMENT;
    for (size_t i = 0; i < input_count + output_count; i++) {
        VxTensorSpec spec = VX_TENSOR_SPEC_INIT;
        spec.name = names[i]; spec.dtype = (VxDataType)dtypes[i]; spec.rank = ranks[i];
        for (uint32_t a = 0; a < ranks[i]; a++) {
            VxDimensionConstraint d = VX_DIMENSION_CONSTRAINT_INIT;
            d.min = d.max = dims[i * VX_MAX_TENSOR_RANK + a];
            spec.dimensions[a] = d;
        }
        specs[i] = spec;
    }
    VxModelSource source = VX_MODEL_SOURCE_INIT;
    source.graph_path = graph_path; source.weight_paths = weight_paths; source.weight_path_count = weight_count;
    VxBackendCompileInput input = VX_BACKEND_COMPILE_INPUT_INIT;
    input.source = &source; input.graph_fingerprint = "sha256:test-graph"; input.shape_domain_proof_identity = "proof:test";
    input.inputs = specs; input.input_count = input_count; input.outputs = specs + input_count; input.output_count = output_count;
    input.packed_arithmetic = (VxPackedArithmetic)packed_arithmetic;
    const char* backends[1] = {policy_name};
    VxBackendPolicy policy = VX_BACKEND_POLICY_INIT;
    policy.mode = VX_BACKEND_REQUIRE; policy.backends = backends; policy.backend_count = 1;
    VxBackendShapeDomainAttestation attestation = VX_BACKEND_SHAPE_DOMAIN_ATTESTATION_INIT;
    fresh_report();
    const VxStatus status = g_provider.compile(g_runtime, &input, &policy, &g_compiled, &attestation, &g_report);
    if (status != VX_STATUS_OK) return (int)status;
    /* what the runtime validates synchronously: echoed identities, attested route, arithmetic */
    if (!attestation.graph_fingerprint || strcmp(attestation.graph_fingerprint, input.graph_fingerprint) ||
        !attestation.shape_domain_proof_identity || strcmp(attestation.shape_domain_proof_identity, input.shape_domain_proof_identity) ||
        !attestation.maximum_tensor_bytes || attestation.maximum_resident_bytes < attestation.maximum_tensor_bytes ||
        !g_report.route_attested || g_report.operator_fallback_used)
        return 1000;
    if (packed_arithmetic == VX_PACKED_ARITHMETIC_DYNAMIC_I8 && attestation.packed_arithmetic != VX_PACKED_ARITHMETIC_UNSPECIFIED &&
        attestation.packed_arithmetic != VX_PACKED_ARITHMETIC_DYNAMIC_I8) return 1001;
    return (int)VX_STATUS_OK;
}

API int fake_host_context_create(int decode_rows) {
    VxContextOptions options = VX_CONTEXT_OPTIONS_INIT;
    if (decode_rows) options.decode_row_mode = (VxDecodeRowMode)1;
    fresh_report();
    return (int)g_provider.context_create(g_compiled, &options, &g_context, &g_report);
}

typedef struct { const char* const* names; void* const* buffers; const size_t* capacity; const uint32_t* dtypes; size_t count; unsigned writes[16]; int bad; } Sink;

static VxStatus sink_write(void* user, const char* name, VxDataType dtype, const int64_t* shape, uint32_t rank, const void* data, size_t bytes) {
    Sink* sink = (Sink*)user;
    for (size_t i = 0; i < sink->count; i++) {
        if (strcmp(sink->names[i], name)) continue;
        size_t elements = 1;
        for (uint32_t a = 0; a < rank; a++) elements *= (size_t)shape[a];
        if (sink->writes[i] || (uint32_t)dtype != sink->dtypes[i] || bytes != sink->capacity[i] || !data || !elements) { sink->bad = 1; return VX_STATUS_INVALID_ARGUMENT; }
        memcpy(sink->buffers[i], data, bytes);   /* copied before write() returns */
        sink->writes[i]++;
        return VX_STATUS_OK;
    }
    sink->bad = 1;
    return VX_STATUS_INVALID_ARGUMENT;
}

/* One execution: bindings by name (HOST), outputs copied by the sink; returns the provider's status, or 2000
 * when an output was missing, duplicated or mistyped. */
API int fake_host_execute(const char* const* in_names, const uint32_t* in_dtypes, const uint32_t* in_ranks, const int64_t* in_dims,
                          const void* const* in_data, const size_t* in_bytes, size_t input_count,
                          const char* const* out_names, const uint32_t* out_dtypes, void* const* out_buffers, const size_t* out_bytes,
                          size_t output_count) {
    VxTensorBinding bindings[16];
    if (input_count > 16 || output_count > 16) return (int)VX_STATUS_INVALID_ARGUMENT;
    for (size_t i = 0; i < input_count; i++) {
        VxTensorBinding b = VX_TENSOR_BINDING_INIT;
        b.name = in_names[i]; b.dtype = (VxDataType)in_dtypes[i]; b.rank = in_ranks[i];
        for (uint32_t a = 0; a < in_ranks[i]; a++) b.shape[a] = in_dims[i * VX_MAX_TENSOR_RANK + a];
        b.data = in_data[i]; b.byte_size = in_bytes[i];
        bindings[i] = b;
    }
    Sink state = {out_names, out_buffers, out_bytes, out_dtypes, output_count, {0}, 0};
    VxBackendOutputSink sink = {sizeof(VxBackendOutputSink), &state, sink_write};
    fresh_report();
    const VxStatus status = g_provider.context_execute(g_context, bindings, input_count, &sink, &g_report);
    if (status != VX_STATUS_OK) return (int)status;
    for (size_t i = 0; i < output_count; i++) if (state.writes[i] != 1) return 2000;
    return state.bad ? 2000 : (int)VX_STATUS_OK;
}

API void fake_host_teardown(void) {
    if (g_context) { if (g_provider.context_close) g_provider.context_close(g_context, &g_report); g_provider.context_destroy(g_context); g_context = NULL; }
    if (g_compiled) { g_provider.compiled_destroy(g_compiled); g_compiled = NULL; }
    if (g_runtime) { g_provider.runtime_destroy(g_runtime); g_runtime = NULL; }
}
API size_t fake_host_max_rank(void) { return VX_MAX_TENSOR_RANK; }
