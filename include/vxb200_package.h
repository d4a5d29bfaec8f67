/*
 * vxb200_package.h - package loader of the B200 W8A8 route: reads a model package
 * (graph.json + SafeTensors files) and runs its W8A8 nodes with activations kept on the
 * device between nodes.
 *
 * What it replaces in the reference: the SafeTensors reader
 * (native/src/runtime/safetensors.c, safetensors_header.c, safetensors_bytes.c), the affine
 * metadata validation of docs/w8a8-safetensors.md:13-121 and docs/model-format.md:280-287, and
 * the per-model one-time weight packing (native/src/runtime/engine_runtime_model.inc:2125-2218).
 * Served operators (everything else makes vxb_package_open decline, so the host keeps the graph
 * on its own routes):
 *   QuantizeLinear / DequantizeLinear / RequantizeLinear with per-tensor metadata,
 *   QLinear   int8 weight [d_out,d_in] (layout dout_din), per-axis axis-0 F32 scales, explicit
 *             all-zero I8 zero points, I32 bias; I8/U8 activations with per-tensor metadata,
 *   PackedLinear  I32 words [N, ceil(K*bits/32)] + F32 scales [N, ceil(K/G)], weight bits 8 or 4,
 *             group size 32/64/128/256, dynamic-I8 arithmetic, fp32 in and out.
 * Return convention as in vxb200_w8a8.h: 1 handled, 0 declined before anything was touched,
 * -1 failed after work was submitted; vxb_last_error() has the reason.
 */
#ifndef VXB200_PACKAGE_H
#define VXB200_PACKAGE_H

#include "vxb200_w8a8.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct VxbPackage VxbPackage; /* parsed graph + tensors mapped from the SafeTensors files (host) */
typedef struct VxbProgram VxbProgram; /* compiled package: repacked weights on the device + the node plan */

/* Tensor dtypes of package inputs and outputs: VXB_DTYPE_U8 / VXB_DTYPE_I8 (vxb200_w8a8.h) and */
#define VXB_DTYPE_F32 18u /* numerically the reference's VX_DTYPE_F32 (native/include/volvoxai_enums.h:492) */
#define VXB_DTYPE_I32 16u /* VX_DTYPE_I32 (:490) */

/* Reads and validates `graph_path` (volvox-graph/v1) and the SafeTensors files.  Validation follows
 * docs/w8a8-safetensors.md "Required validation": exact format string, every reference resolves
 * uniquely, dtypes / ranks / counts of scales and zero points match their targets, scales finite
 * and positive, Q/DQ operands identical to the central descriptors; nothing is coerced or guessed. */
VXB_API int vxb_package_open(const char* graph_path, const char* const* weight_paths, size_t weight_path_count,
                     VxbPackage** out);
VXB_API void vxb_package_close(VxbPackage* package);
VXB_API uint32_t vxb_package_node_count(const VxbPackage* package);
/* "QLinear", "PackedLinear", ...; NULL when index is out of range. */
VXB_API const char* vxb_package_node_op(const VxbPackage* package, uint32_t index);
/* Graph inputs (is_output == 0) or outputs (is_output != 0), in declaration order. */
VXB_API uint32_t vxb_package_io_count(const VxbPackage* package, int is_output);
VXB_API const char* vxb_package_io_name(const VxbPackage* package, int is_output, uint32_t index);
VXB_API uint32_t vxb_package_io_dtype(const VxbPackage* package, int is_output, uint32_t index);
VXB_API uint32_t vxb_package_io_rank(const VxbPackage* package, int is_output, uint32_t index);
VXB_API int64_t vxb_package_io_dim(const VxbPackage* package, int is_output, uint32_t index, uint32_t axis);
VXB_API uint64_t vxb_package_io_bytes(const VxbPackage* package, int is_output, uint32_t index);

/* Uploads and repacks every weight once (the compile-time step) and allocates the device buffers
 * of all intermediate tensors.  The program borrows nothing from the package afterwards. */
VXB_API int vxb_program_compile(VxbContext* ctx, const VxbPackage* package, VxbProgram** out);
VXB_API void vxb_program_destroy(VxbProgram* program);
VXB_API uint64_t vxb_program_device_bytes(const VxbProgram* program);
/* "node-id=route;..." of the last execute, e.g. "projection=static+decode-rows-tcgen05-i8+e2". */
VXB_API const char* vxb_program_route_evidence(const VxbProgram* program);

/* One forward pass.  inputs[i] / outputs[i] are HOST buffers in the package's declaration order with
 * exactly vxb_package_io_bytes() bytes each.  Inputs are uploaded once, every node runs on the
 * device on the context's stream, outputs are downloaded, and the call returns when they are in
 * place: intermediate tensors never cross PCIe. */
VXB_API int vxb_program_execute(VxbProgram* program, const void* const* inputs, const size_t* input_bytes,
                        uint32_t input_count, void* const* outputs, const size_t* output_bytes,
                        uint32_t output_count);

#ifdef __cplusplus
}
#endif
#endif /* VXB200_PACKAGE_H */
