/*
 * Drop-in harness (TEST INFRASTRUCTURE, not shipped): a minimal Dataflow_Handle built on the reference's own
 * headers, op table and fingerprinting, so that the reference's own submitters
 * (dataflow_submit_default_select_experts, ..., dataflow_submit_matmul - compiled from the reference sources
 * next to this file, see ../Makefile target `dropin`) dispatch into the B200 external-op adapter exactly as
 * backends/nvidia/src/handle/src/cuda_dataflow_handle.c would: fingerprint lookup in the op table, then a call of
 * the registered external function with (handle, stream_id, op, op_extra).
 * Only the pieces an external op needs are filled in: one stream, the op table, submit_op and
 * register_external_code. Everything else of the vtable stays NULL.
 */
#include <dlfcn.h>

#include "dataflow_ops.h"
#include "cuda_dataflow_handle.h"

/* dataflow_datatype.c refers to the bulk conversion routines; nothing on this path calls them, and their
 * AVX-512 sources are not built here. These placeholders only satisfy the dynamic linker. */
void convert_datatype(void) {}
void convert_datatype_avx512(void) {}

static uint64_t harness_hash(void * fingerprint, uint64_t table_size) {
	/* least significant 8 bytes of the fingerprint, as the reference's handle does
	 * (cuda_dataflow_handle.c:30-44) */
	uint8_t * tail = ((uint8_t *) fingerprint) + DATAFLOW_OP_IDENTIFIER_FINGERPRINT_NUM_BYTES - sizeof(uint64_t);
	uint64_t v = 0;
	for (int i = 0; i < 8; i++) {
		v = (v << 8) | (uint64_t) tail[i];
	}
	return v % table_size;
}

static int harness_get_num_procs(Dataflow_Handle * handle) {
	return 0;
}

static int harness_register_external_code(Dataflow_Handle * handle, char * so_path, int num_funcs, Op_Skeleton * skeletons,
											char ** symbols, char ** init_symbols) {
	void * lib = dlopen(so_path, RTLD_LAZY | RTLD_GLOBAL);
	if (!lib) {
		fprintf(stderr, "harness: dlopen(%s) failed: %s\n", so_path, dlerror());
		return -1;
	}
	int added = 0;
	for (int i = 0; i < num_funcs; i++) {
		Cuda_Function fn;
		memset(&fn, 0, sizeof(fn));
		fn.cuda_external_func = dlsym(lib, symbols[i]);
		if (!fn.cuda_external_func) {
			fprintf(stderr, "harness: symbol %s missing in %s\n", symbols[i], so_path);
			continue;
		}
		if (init_symbols && init_symbols[i]) {
			External_Lib_Func_Init init = dlsym(lib, init_symbols[i]);
			if (!init || init(handle, &fn)) {
				continue;
			}
		}
		fn.is_native = false;
		memcpy(&fn.op_skeleton, &skeletons[i], sizeof(Op_Skeleton));
		if (dataflow_insert_table(&(handle -> op_table), fn.op_skeleton.identifier.fingerprint, &fn)) {
			fprintf(stderr, "harness: could not insert %s (duplicate fingerprint?)\n", symbols[i]);
			continue;
		}
		added++;
	}
	handle -> num_ops += added;
	return added;
}

static int harness_submit_op(Dataflow_Handle * handle, Op * op, int stream_id) {
	Cuda_Function * fn = NULL;
	long ind = dataflow_find_table(&(handle -> op_table), (op -> op_skeleton).identifier.fingerprint, false, (void **) &fn);
	if (ind == -1 || !fn) {
		fprintf(stderr, "harness: no op registered for %s\n", (op -> op_skeleton).header.op_nickname);
		return -1;
	}
	return (fn -> cuda_external_func)(handle, stream_id, op, fn -> op_extra);
}

/* stream: the CUstream / cudaStream_t ops are submitted to (stream id 0). Returns NULL on failure. */
Dataflow_Handle * dropin_create_handle(void * stream, char * adapter_so_path) {
	Dataflow_Handle * h = calloc(1, sizeof(Dataflow_Handle));
	if (!h) return NULL;
	h -> compute_type = COMPUTE_CUDA;
	h -> num_streams = 1;
	CUstream * streams = malloc(sizeof(CUstream));
	streams[0] = (CUstream) stream;
	h -> streams = streams;
	h -> get_num_procs = harness_get_num_procs;
	h -> register_external_code = harness_register_external_code;
	h -> submit_op = harness_submit_op;
	if (dataflow_init_table(&(h -> op_table), &harness_hash, DATAFLOW_OP_IDENTIFIER_FINGERPRINT_NUM_BYTES, sizeof(Cuda_Function),
							OP_TABLE_MIN_SIZE, OP_TABLE_MAX_SIZE, 1.0f, 1.0f)) {
		return NULL;
	}
	void * lib = dlopen(adapter_so_path, RTLD_LAZY | RTLD_GLOBAL);
	if (!lib) {
		fprintf(stderr, "harness: dlopen(%s) failed: %s\n", adapter_so_path, dlerror());
		return NULL;
	}
	int (*reg)(Dataflow_Handle *, char *) = dlsym(lib, "dataflow_register_b200_moe_ops");
	if (!reg || reg(h, adapter_so_path) < 0) {
		fprintf(stderr, "harness: registration of the B200 MoE ops failed\n");
		return NULL;
	}
	return h;
}

int dropin_num_ops(Dataflow_Handle * h) {
	return h -> num_ops;
}
