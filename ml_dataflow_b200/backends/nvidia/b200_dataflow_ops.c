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
 * Three additive ops (all experts of one pass per call) come with their own skeleton setters and submitters.
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

/* ------------------------------------------------------------------------------------------------------------
 * Additive grouped ops. The reference expresses the experts as a host loop of single matmuls around a stream
 * sync (libdataflowmodels/src/transformer/src/dataflow_transformer.c:2789, 2848-2940, 3460-3641, 4101-4148); these
 * three ops run all experts of one pass in two or three launches and read the per-expert row counts on the device.
 * They are new skeletons in the reference's own style (libdataflowops/src/set_ops/set_op_skeletons.c:1087-1122):
 * nickname "<op>_<dtype>", scalar and buffer argument dtypes, SHA-256 fingerprint of the header - and new
 * submitters in the style of libdataflowops/src/submit_ops/moe_ops.c, so a caller reaches them through
 * handle->submit_op like every other op.
 * ------------------------------------------------------------------------------------------------------------ */

static void set_grouped_skeleton(Op_Skeleton * skeleton, const char * name, DataflowDatatype dt, int num_args,
									const DataflowDatatype * dtypes) {
	Op_Skeleton_Header * header = &(skeleton -> header);
	memset(header, 0, sizeof(Op_Skeleton_Header));
	snprintf(header -> op_nickname, MAX_OP_NICKNAME_SIZE, "%s_%s", name, dataflow_datatype_as_string(dt));
	header -> num_args = num_args;
	for (int i = 0; i < MAX_OP_ARGS; i++) {
		(header -> arg_dtypes)[i] = i < num_args ? dtypes[i] : DATAFLOW_NONE;
	}
	dataflow_do_fingerprinting(header, sizeof(Op_Skeleton_Header), (skeleton -> identifier).fingerprint);
}

#define I_S DATAFLOW_INT_SCALAR
#define L_S DATAFLOW_LONG_SCALAR

/* args: total_rows, model_dim, ffn_dim, num_experts, zone, W1, W3, W2, w1/w3/w2 expert strides (elements),
 * expert_counts, expert_counts_cumsum (inclusive), x1, x3, h, Y */
void dataflow_set_b200_moe_experts_fwd_skeleton(Op_Skeleton * skeleton, DataflowDatatype dt) {
	DataflowDatatype a[17] = {I_S, I_S, I_S, I_S, dt, dt, dt, dt, L_S, L_S, L_S, DATAFLOW_INT, DATAFLOW_INT, dt, dt, dt, dt};
	set_grouped_skeleton(skeleton, "b200_moe_experts_fwd", dt, 17, a);
}

/* args: total_rows, model_dim, ffn_dim, num_experts, dY_zone, row_weights, x1, x3, W1, W3, W2, strides x3,
 * expert_counts, expert_counts_cumsum, dx1, dx3, hs (may be NULL), dP (fp32, caller zeroes), dZ */
void dataflow_set_b200_moe_experts_bwd_x_skeleton(Op_Skeleton * skeleton, DataflowDatatype dt) {
	DataflowDatatype a[21] = {I_S, I_S, I_S, I_S, dt, DATAFLOW_FP32, dt, dt, dt, dt, dt, L_S, L_S, L_S, DATAFLOW_INT,
								DATAFLOW_INT, dt, dt, dt, DATAFLOW_FP32, dt};
	set_grouped_skeleton(skeleton, "b200_moe_experts_bwd_x", dt, 21, a);
}

/* args: total_rows, model_dim, ffn_dim, num_experts, dY_zone, hs, zone_x, dx1, dx3, dW1, dW3, dW2 (each may be
 * NULL), strides x3, expert_counts, expert_counts_cumsum */
void dataflow_set_b200_moe_experts_bwd_w_skeleton(Op_Skeleton * skeleton, DataflowDatatype dt) {
	DataflowDatatype a[17] = {I_S, I_S, I_S, I_S, dt, dt, dt, dt, dt, dt, dt, dt, L_S, L_S, L_S, DATAFLOW_INT, DATAFLOW_INT};
	set_grouped_skeleton(skeleton, "b200_moe_experts_bwd_w", dt, 17, a);
}

int b200_ext_moe_experts_fwd(Dataflow_Handle * handle, int stream_id, Op * op, void * op_extra) {
	void * s;
	if (stream_of(handle, stream_id, &s, "moe_experts_fwd") || require_bf16(op, 4, "moe_experts_fwd")) return -1;
	return b200_moe_experts_fwd(ARG(int, 0), ARG(int, 1), ARG(int, 2), ARG(int, 3), ARG(void *, 4), ARG(void *, 5),
		ARG(void *, 6), ARG(void *, 7), ARG(int64_t, 8), ARG(int64_t, 9), ARG(int64_t, 10), ARG(int *, 11), ARG(int *, 12),
		ARG(void *, 13), ARG(void *, 14), ARG(void *, 15), ARG(void *, 16), s);
}

int b200_ext_moe_experts_bwd_x(Dataflow_Handle * handle, int stream_id, Op * op, void * op_extra) {
	void * s;
	if (stream_of(handle, stream_id, &s, "moe_experts_bwd_x") || require_bf16(op, 4, "moe_experts_bwd_x")) return -1;
	return b200_moe_experts_bwd_x(ARG(int, 0), ARG(int, 1), ARG(int, 2), ARG(int, 3), ARG(void *, 4), ARG(float *, 5),
		ARG(void *, 6), ARG(void *, 7), ARG(void *, 8), ARG(void *, 9), ARG(void *, 10), ARG(int64_t, 11), ARG(int64_t, 12),
		ARG(int64_t, 13), ARG(int *, 14), ARG(int *, 15), ARG(void *, 16), ARG(void *, 17), ARG(void *, 18), ARG(float *, 19),
		ARG(void *, 20), s);
}

int b200_ext_moe_experts_bwd_w(Dataflow_Handle * handle, int stream_id, Op * op, void * op_extra) {
	void * s;
	if (stream_of(handle, stream_id, &s, "moe_experts_bwd_w") || require_bf16(op, 4, "moe_experts_bwd_w")) return -1;
	return b200_moe_experts_bwd_w(ARG(int, 0), ARG(int, 1), ARG(int, 2), ARG(int, 3), ARG(void *, 4), ARG(void *, 5),
		ARG(void *, 6), ARG(void *, 7), ARG(void *, 8), ARG(void *, 9), ARG(void *, 10), ARG(void *, 11), ARG(int64_t, 12),
		ARG(int64_t, 13), ARG(int64_t, 14), ARG(int *, 15), ARG(int *, 16), s);
}

int dataflow_submit_b200_moe_experts_fwd(Dataflow_Handle * handle, int stream_id, DataflowDatatype dt,
		int total_rows, int model_dim, int ffn_dim, int num_experts, void * zone, void * W1, void * W3, void * W2,
		int64_t w1_stride_elems, int64_t w3_stride_elems, int64_t w2_stride_elems, int * expert_counts,
		int * expert_counts_cumsum, void * x1, void * x3, void * h, void * Y) {
	Op op;
	dataflow_set_b200_moe_experts_fwd_skeleton(&op.op_skeleton, dt);
	void ** a = op.op_args;
	a[0] = &total_rows; a[1] = &model_dim; a[2] = &ffn_dim; a[3] = &num_experts; a[4] = &zone; a[5] = &W1; a[6] = &W3;
	a[7] = &W2; a[8] = &w1_stride_elems; a[9] = &w3_stride_elems; a[10] = &w2_stride_elems; a[11] = &expert_counts;
	a[12] = &expert_counts_cumsum; a[13] = &x1; a[14] = &x3; a[15] = &h; a[16] = &Y;
	if ((handle -> submit_op)(handle, &op, stream_id)) {
		fprintf(stderr, "Error: failed to submit b200 moe experts fwd op...\n");
		return -1;
	}
	return 0;
}

int dataflow_submit_b200_moe_experts_bwd_x(Dataflow_Handle * handle, int stream_id, DataflowDatatype dt,
		int total_rows, int model_dim, int ffn_dim, int num_experts, void * dY_zone, float * row_weights, void * x1,
		void * x3, void * W1, void * W3, void * W2, int64_t w1_stride_elems, int64_t w3_stride_elems,
		int64_t w2_stride_elems, int * expert_counts, int * expert_counts_cumsum, void * dx1, void * dx3, void * hs,
		float * dP, void * dZ) {
	Op op;
	dataflow_set_b200_moe_experts_bwd_x_skeleton(&op.op_skeleton, dt);
	void ** a = op.op_args;
	a[0] = &total_rows; a[1] = &model_dim; a[2] = &ffn_dim; a[3] = &num_experts; a[4] = &dY_zone; a[5] = &row_weights;
	a[6] = &x1; a[7] = &x3; a[8] = &W1; a[9] = &W3; a[10] = &W2; a[11] = &w1_stride_elems; a[12] = &w3_stride_elems;
	a[13] = &w2_stride_elems; a[14] = &expert_counts; a[15] = &expert_counts_cumsum; a[16] = &dx1; a[17] = &dx3;
	a[18] = &hs; a[19] = &dP; a[20] = &dZ;
	if ((handle -> submit_op)(handle, &op, stream_id)) {
		fprintf(stderr, "Error: failed to submit b200 moe experts bwd_x op...\n");
		return -1;
	}
	return 0;
}

int dataflow_submit_b200_moe_experts_bwd_w(Dataflow_Handle * handle, int stream_id, DataflowDatatype dt,
		int total_rows, int model_dim, int ffn_dim, int num_experts, void * dY_zone, void * hs, void * zone_x, void * dx1,
		void * dx3, void * dW1, void * dW3, void * dW2, int64_t dw1_stride_elems, int64_t dw3_stride_elems,
		int64_t dw2_stride_elems, int * expert_counts, int * expert_counts_cumsum) {
	Op op;
	dataflow_set_b200_moe_experts_bwd_w_skeleton(&op.op_skeleton, dt);
	void ** a = op.op_args;
	a[0] = &total_rows; a[1] = &model_dim; a[2] = &ffn_dim; a[3] = &num_experts; a[4] = &dY_zone; a[5] = &hs;
	a[6] = &zone_x; a[7] = &dx1; a[8] = &dx3; a[9] = &dW1; a[10] = &dW3; a[11] = &dW2; a[12] = &dw1_stride_elems;
	a[13] = &dw3_stride_elems; a[14] = &dw2_stride_elems; a[15] = &expert_counts; a[16] = &expert_counts_cumsum;
	if ((handle -> submit_op)(handle, &op, stream_id)) {
		fprintf(stderr, "Error: failed to submit b200 moe experts bwd_w op...\n");
		return -1;
	}
	return 0;
}

#define B200_NUM_EXT_OPS 15

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
	dataflow_set_b200_moe_experts_fwd_skeleton(&sk[n], DATAFLOW_BF16); syms[n++] = "b200_ext_moe_experts_fwd";
	dataflow_set_b200_moe_experts_bwd_x_skeleton(&sk[n], DATAFLOW_BF16); syms[n++] = "b200_ext_moe_experts_bwd_x";
	dataflow_set_b200_moe_experts_bwd_w_skeleton(&sk[n], DATAFLOW_BF16); syms[n++] = "b200_ext_moe_experts_bwd_w";

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
