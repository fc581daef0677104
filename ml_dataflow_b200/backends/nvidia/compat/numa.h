/* Stand-in for <numa.h> on build hosts without libnuma development files.
 * The reference's libdataflow/include/dataflow_common.h includes <numa.h>, but nothing the
 * MoE op adapter touches uses a libnuma symbol. Put this directory on the include path only
 * when the system header is missing. */
#ifndef B200_COMPAT_NUMA_H
#define B200_COMPAT_NUMA_H
#endif
