/*
 * External-op adapter: the B200 MoE kernels behind ml_dataflow's own op dispatch.
 *
 * Compiled against the reference's headers where they lie (nothing is copied):
 *   -I$REF/libdataflow/include -I$REF/libdataflowops/include -I$REF/backends/nvidia/include
 * Every function below has the reference's external-op signature
 *   int fn(Dataflow_Handle *, int stream_id, Op *, void *op_extra)      (dataflow_handle.h:166)
 * and unpacks op->op_args - pointers to the argument values, in the parameter order of the matching
 * dataflow_submit_* function (libdataflowops/src/submit_ops/moe_ops.c, matmul_op.c, mlp_misc_ops.c) -
 * into the C ABI of include/b200_moe.h. dataflow_register_b200_moe_ops() registers them under the same
 * op skeletons the submitters build, so libdataflowmodels' MoE block reaches these kernels unchanged.
 */
#include "dataflow_ops.h"
#include "cuda_dataflow_handle.h"

#include "b200_moe.h"

#define ARG(type, i) (*(type *) (op -> op_args[(i)]))

/* stream_id indexes handle->streams (CUstream[]); like cublas_matmul
 * (backends/nvidia/src/ops/src/external/matmul_helper/src/matmul_helper.c:788-795) reject ids out of range. */
static int stream_of(Dataflow_Handle * handle, int stream_id, void ** stream_out, const char * op_name) {
	if (stream_id < 0 || stream_id >= handle -> num_streams) {
		fprintf(stderr, "Error: %s: stream id %d out of range (handle has %d streams)...\n", op_name, stream_id, handle -> num_streams);
		return -1;
	}
	*stream_out = (void *) (((CUstream *) (handle -> streams))[stream_id]);
	return 0;
}

static int arg_dt(Op * op, int i) {
	return (int) (op -> op_skeleton).header.arg_dtypes[i];
}

static int require_bf16(Op * op, int i, const char * op_name) {
	if (arg_dt(op, i) != DATAFLOW_BF16) {
		fprintf(stderr, "Error: %s: only bf16 tensors are implemented on this backend (argument %d has dtype %s)...\n",
			op_name, i, dataflow_datatype_as_string((DataflowDatatype) arg_dt(op, i)));
		return -1;
	}
	return 0;
}

int b200_ext_select_experts(Dataflow_Handle * handle, int stream_id, Op * op, void * op_extra) {
	void * s;
	if (stream_of(handle, stream_id, &s, "select_experts")) return -1;
	return b200_select_experts(arg_dt(op, 3), ARG(int, 0), ARG(int, 1), ARG(int, 2), ARG(void *, 3), ARG(float *, 4),
		ARG(uint16_t *, 5), ARG(int *, 6), ARG(int *, 7), ARG(int *, 8), s);
}

int b200_ext_build_expert_mapping(Dataflow_Handle * handle, int stream_id, Op * op, void * op_extra) {
	void * s;
	if (stream_of(handle, stream_id, &s, "build_expert_mapping")) return -1;
	/* seven arguments and no workspace in the op signature, no allocation at submit time: the kernel's
	 * tables live in the library's built-in scratch array */
	return b200_build_expert_mapping_static(ARG(int, 0), ARG(int, 1), ARG(int, 2), ARG(uint16_t *, 3), ARG(int *, 4),
		ARG(int *, 5), ARG(int *, 6), s);
}

int b200_ext_prepare_experts(Dataflow_Handle * handle, int stream_id, Op * op, void * op_extra) {
	void * s;
	if (stream_of(handle, stream_id, &s, "prepare_experts") || require_bf16(op, 3, "prepare_experts") || require_bf16(op, 5, "prepare_experts")) return -1;
	return b200_prepare_experts(ARG(int, 0), ARG(int, 1), ARG(int, 2), ARG(void *, 3), ARG(int *, 4), ARG(void *, 5), s);
}

int b200_ext_prepare_expert_zone(Dataflow_Handle * handle, int stream_id, Op * op, void * op_extra) {
	void * s;
	if (stream_of(handle, stream_id, &s, "prepare_expert_zone") || require_bf16(op, 1, "prepare_expert_zone") || require_bf16(op, 6, "prepare_expert_zone")) return -1;
	return b200_prepare_expert_zone(ARG(int, 0), ARG(void *, 1), ARG(int, 2), ARG(int *, 3), ARG(int *, 4), ARG(int *, 5),
		ARG(void *, 6), s);
}

int b200_ext_merge_experts(Dataflow_Handle * handle, int stream_id, Op * op, void * op_extra) {
	void * s;
	if (stream_of(handle, stream_id, &s, "merge_experts") || require_bf16(op, 3, "merge_experts") || require_bf16(op, 6, "merge_experts")) return -1;
	return b200_merge_experts(ARG(int, 0), ARG(int, 1), ARG(int, 2), ARG(void *, 3), ARG(int *, 4), ARG(float *, 5),
		ARG(void *, 6), s);
}

int b200_ext_merge_expert_result(Dataflow_Handle * handle, int stream_id, Op * op, void * op_extra) {
	void * s;
	if (stream_of(handle, stream_id, &s, "merge_expert_result") || require_bf16(op, 3, "merge_expert_result") || require_bf16(op, 9, "merge_expert_result")) return -1;
	return b200_merge_expert_result(ARG(int, 0), ARG(int, 1), ARG(int, 2), ARG(void *, 3), ARG(int, 4), ARG(int *, 5),
		ARG(int *, 6), ARG(float *, 7), ARG(uint16_t *, 8), ARG(void *, 9), s);
}

int b200_ext_router_bwd_x(Dataflow_Handle * handle, int stream_id, Op * op, void * op_extra) {
	void * s;
	if (stream_of(handle, stream_id, &s, "router_bwd_x") || require_bf16(op, 9, "router_bwd_x") || require_bf16(op, 10, "router_bwd_x")) return -1;
	return b200_router_bwd_x(ARG(int, 0), ARG(int, 1), ARG(int, 2), ARG(int, 3), ARG(int, 4), ARG(int *, 5), ARG(int *, 6),
		ARG(uint16_t *, 7), ARG(float *, 8), ARG(void *, 9), ARG(void *, 10), ARG(void *, 11), ARG(void *, 12), s);
}

int b200_ext_router_gate_bwd_x(Dataflow_Handle * handle, int stream_id, Op * op, void * op_extra) {
	void * s;
	if (stream_of(handle, stream_id, &s, "router_gate_bwd_x") || require_bf16(op, 5, "router_gate_bwd_x")) return -1;
	return b200_router_gate_bwd_x(ARG(int, 0), ARG(int, 1), ARG(int, 2), ARG(uint16_t *, 3), ARG(float *, 4), ARG(void *, 5), s);
}

int b200_ext_swiglu(Dataflow_Handle * handle, int stream_id, Op * op, void * op_extra) {
	void * s;
	if (stream_of(handle, stream_id, &s, "swiglu") || require_bf16(op, 2, "swiglu")) return -1;
	return b200_swiglu(ARG(int, 0), ARG(int, 1), ARG(void *, 2), ARG(void *, 3), ARG(void *, 4), s);
}

int b200_ext_swiglu_bwd_x(Dataflow_Handle * handle, int stream_id, Op * op, void * op_extra) {
	void * s;
	if (stream_of(handle, stream_id, &s, "swiglu_bwd_x") || require_bf16(op, 2, "swiglu_bwd_x") || require_bf16(op, 4, "swiglu_bwd_x")) return -1;
	return b200_swiglu_bwd_x(ARG(int, 0), ARG(int, 1), ARG(void *, 2), ARG(void *, 3), ARG(void *, 4), ARG(void *, 5),
		ARG(void *, 6), s);
}

/* matmul: 19 arguments (libdataflowops/src/submit_ops/matmul_op.c:33-53); argument 0 is the SM budget, which
 * these persistent kernels ignore (they size their grid from the device). */
int b200_ext_matmul(Dataflow_Handle * handle, int stream_id, Op * op, void * op_extra) {
	void * s;
	if (stream_of(handle, stream_id, &s, "matmul")) return -1;
	return b200_matmul((int) ARG(DataflowDatatype, 1), (int) ARG(DataflowDatatype, 2), (int) ARG(DataflowDatatype, 3),
		(int) ARG(DataflowDatatype, 4), ARG(int, 6), ARG(int, 7), ARG(int, 8), ARG(int, 9), ARG(int, 10),
		ARG(float, 11), ARG(float, 12), ARG(void *, 13), ARG(void *, 14), ARG(void *, 15), ARG(void *, 16),
		ARG(uint64_t, 17), ARG(void *, 18), s);
}

#define B200_NUM_EXT_OPS 12

/*
 * Registers the external ops above with `handle` from the shared library at `adapter_so_path` (this file's
 * own .so). Call it instead of, or before, dataflow_register_default_ops(): the op table refuses a
 * fingerprint that is already present (libdataflow/src/dataflow_table/dataflow_table.c:398-413).
 * Returns the number of ops registered, or -1.
 */
int dataflow_register_b200_moe_ops(Dataflow_Handle * handle, char * adapter_so_path) {
	Op_Skeleton sk[B200_NUM_EXT_OPS];
	char * syms[B200_NUM_EXT_OPS];
	char * inits[B200_NUM_EXT_OPS];
	int n = 0;

	dataflow_set_default_select_experts_skeleton(&sk[n], DATAFLOW_FP32); syms[n++] = "b200_ext_select_experts";
	dataflow_set_default_select_experts_skeleton(&sk[n], DATAFLOW_BF16); syms[n++] = "b200_ext_select_experts";
	dataflow_set_default_build_expert_mapping_skeleton(&sk[n]); syms[n++] = "b200_ext_build_expert_mapping";
	dataflow_set_default_prepare_experts_skeleton(&sk[n], DATAFLOW_BF16, DATAFLOW_BF16); syms[n++] = "b200_ext_prepare_experts";
	dataflow_set_default_prepare_expert_zone_skeleton(&sk[n], DATAFLOW_BF16, DATAFLOW_BF16); syms[n++] = "b200_ext_prepare_expert_zone";
	dataflow_set_default_merge_experts_skeleton(&sk[n], DATAFLOW_BF16, DATAFLOW_BF16); syms[n++] = "b200_ext_merge_experts";
	dataflow_set_default_merge_expert_result_skeleton(&sk[n], DATAFLOW_BF16, DATAFLOW_BF16); syms[n++] = "b200_ext_merge_expert_result";
	dataflow_set_default_router_bwd_x_skeleton(&sk[n], DATAFLOW_BF16, DATAFLOW_BF16); syms[n++] = "b200_ext_router_bwd_x";
	dataflow_set_default_router_gate_bwd_x_skeleton(&sk[n], DATAFLOW_BF16, DATAFLOW_BF16); syms[n++] = "b200_ext_router_gate_bwd_x";
	dataflow_set_default_swiglu_skeleton(&sk[n], DATAFLOW_BF16); syms[n++] = "b200_ext_swiglu";
	dataflow_set_default_swiglu_bwd_x_skeleton(&sk[n], DATAFLOW_BF16, DATAFLOW_BF16); syms[n++] = "b200_ext_swiglu_bwd_x";
	dataflow_set_matmul_skeleton(&sk[n]); syms[n++] = "b200_ext_matmul";

	for (int i = 0; i < n; i++) {
		inits[i] = NULL;
	}

	int added = (handle -> register_external_code)(handle, adapter_so_path, n, sk, syms, inits);
	if (added != n) {
		fprintf(stderr, "Error: registered %d of %d B200 MoE ops from %s...\n", added, n, adapter_so_path);
		return -1;
	}
	return added;
}
