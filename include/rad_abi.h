/* rad_abi.h -- clean-room stand-in for the radiance engine's kernel-plugin ABI.
 *
 * The real header belongs to the radiance engine and is not shipped with libr3d.
 * Everything here is reconstructed from how libr3d USES the ABI:
 *   - struct field order from positional initialisers
 *       RadTensor   tools/probe_m4_entry.cpp:48-55
 *       RadArgs     tools/probe_m4_entry.cpp:59
 *       RadParam    tools/replay_dump.cpp:198-199
 *       RadKernelInfo / RadConstraint / RadOpSchema   src/r3d_rows.cpp:793-1036, :1425-1433
 *   - enumerator NAMES from src/r3d_rows.cpp and the three gemm entries.
 * What cannot be recovered is marked UNPINNED: numeric enumerator values, the maximum
 * tensor rank, and struct packing beyond natural alignment. A maintainer who owns the
 * real header drops it in place of this file and rebuilds; no other file spells a number.
 *
 * ABI version: pinned to the value the reference is built against (README.md:10).
 */
#ifndef RAD_ABI_H
#define RAD_ABI_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RAD_ABI_VERSION 26u

/* ---- status codes (names: src/r3d_gemm_fp8a8.hip:829-836). Values UNPINNED. ---- */
enum {
    RAD_OK            = 0,
    RAD_E_INVAL       = 1,
    RAD_E_UNSUPPORTED = 2,
    RAD_E_SHAPE       = 3,
    RAD_E_STRIDE      = 4,
    RAD_E_DTYPE       = 5,
    RAD_E_DEVICE      = 6
};

/* ---- element types used on the quantised-matmul path. Values UNPINNED. ---- */
enum {
    RAD_F32     = 1,
    RAD_F16     = 2,
    RAD_BF16    = 3,
    RAD_F8E4M3  = 4,
    RAD_F8E5M2  = 5,
    RAD_FP4E2M1 = 6,
    RAD_E8M0    = 7,
    RAD_U8      = 8,
    RAD_I8      = 9,
    RAD_I32     = 10,
    RAD_I64     = 11,
    RAD_U4      = 12,
    RAD_U2      = 13,
    RAD_F64     = 14
};

#define RAD_MAX_RANK 8   /* UNPINNED */

/* Strides are in ELEMENTS, not bytes (tools/probe_m4_entry.cpp:52). A packed fp4 tensor's
 * shape counts elements; its storage is shape/2 bytes per row. */
typedef struct RadTensor {
    void*    data;
    uint32_t dtype;
    uint32_t rank;
    int64_t  shape[RAD_MAX_RANK];
    int64_t  stride[RAD_MAX_RANK];
} RadTensor;

enum { RAD_PK_INT = 0, RAD_PK_F64 = 1, RAD_PK_STR = 2 };   /* RadParam.kind, UNPINNED */

typedef struct RadParam {
    const char* key;
    int         kind;
    long long   ival;
    long long   ihi;
    const char* sval;
    double      dval;
} RadParam;

#define RAD_INT(k, v) { (k), RAD_PK_INT, (long long)(v), 0, NULL, 0.0 }
#define RAD_F64V(k, v) { (k), RAD_PK_F64, 0, 0, NULL, (double)(v) }
#define RAD_STR(k, v) { (k), RAD_PK_STR, 0, 0, (v), 0.0 }

typedef struct RadArgs {
    RadTensor* t;
    int        n_t;
    RadParam*  p;
    int        n_p;
    void*      scratch;
    int64_t    scratch_bytes;
    void*      reserved0;
    int        reserved1;
    int        reserved2;
} RadArgs;

/* Opaque stream handle; a CUDA plugin reads it as (cudaStream_t)(uintptr_t)s, the way the
 * reference reads a hipStream_t (src/r3d_gemm_fp8a8.hip:942). */
typedef void* RadStream;

/* ---- plugin identity (src/r3d_rows.cpp:18-27) ---- */
enum { RAD_PLUGIN_KERNEL = 1 };
typedef struct RadPluginInfo {
    int         kind;
    const char* name;
    const char* version;
    const char* description;
    const char* targets;
} RadPluginInfo;

/* ---- op schemas (src/r3d_rows.cpp:190-245) ---- */
enum { RAD_P_INT = 0, RAD_P_F64 = 1, RAD_P_STR = 2 };
enum { RAD_REQUIRED = 0, RAD_OPTIONAL = 1, RAD_DERIVED = 2 };
enum { RAD_OPD_IN = 0, RAD_OPD_OUT = 1, RAD_OPD_INOUT = 2, RAD_OPD_WEIGHT = 3 };

typedef struct RadParamSpec {
    const char* name;
    int         type;
    int         need;
    int         role;
} RadParamSpec;

typedef struct RadOperandSpec {
    const char* name;
    int         dir;
    int         optional;
} RadOperandSpec;

typedef struct RadOpSchema {
    const char*           op;
    const RadParamSpec*   params;
    int                   n_params;
    const RadOperandSpec* operands;
    int                   n_operands;
    const char*           doc;
} RadOpSchema;

/* ---- kernel rows (src/r3d_rows.cpp:1033-1036, :1588-1599) ---- */
enum { RAD_C_EQ = 0, RAD_C_LE = 1, RAD_C_GE = 2, RAD_C_DIV = 3, RAD_C_IN = 4 };
enum { RAD_DOMAIN_HOST = 0, RAD_DOMAIN_DEVICE = 1 };

/* A constraint on a key the query does not carry does not hold
 * (src/r3d_rows.cpp:1105-1110). RAD_C_IN matches one word of a space-separated list. */
typedef struct RadConstraint {
    const char* key;
    int         op;
    long long   ival;
    const char* sval;
} RadConstraint;

typedef struct RadTunable {
    const char* key;
    long long   lo, hi, def;
} RadTunable;

/* ---- weight encodings and layout hooks (src/r3d_gemm_logits.hip:233-272) ---- */
#define RAD_ENC_STR        16   /* UNPINNED */
#define RAD_ENC_MAX_PLANES 4    /* UNPINNED */
enum { RAD_PLANE_TILED = 1 };

typedef struct RadEncPlane {
    char     role[RAD_ENC_STR];
    int      kind;
    uint32_t dtype;
    int64_t  block[2];
} RadEncPlane;

typedef struct RadEncoding {
    char        scheme[RAD_ENC_STR];
    int         n_planes;
    char        transform[RAD_ENC_STR];
    RadEncPlane plane[RAD_ENC_MAX_PLANES];
} RadEncoding;

typedef struct RadLayout {
    int64_t     bytes;
    int64_t     align;
    const char* tag;
} RadLayout;

typedef int     (*RadLaunchFn)(const RadArgs*, RadStream);
typedef int64_t (*RadScratchFn)(const RadArgs*);
typedef int     (*RadInitFn)(void);
typedef void    (*RadFiniFn)(void);
typedef int     (*RadLayoutFn)(const RadParam*, int, int, const RadEncoding*, const int*,
                               const RadTensor*, int, RadLayout*);
typedef int     (*RadRelayoutFn)(const RadParam*, int, int, const RadEncoding*, const int*,
                                 const RadTensor*, int, void*, int64_t);
typedef int     (*RadOpdShapeFn)(const RadParam*, int, int, RadTensor*);
typedef int     (*RadUnrelayoutFn)(const RadParam*, int, int, const RadEncoding*, const int*,
                                   const void*, int64_t, const RadTensor*, int);

typedef struct RadKernelInfo {
    const char*          name;
    const char*          op;
    const char*          family;
    const char*          summary;
    const char*          shapes;
    const char*          dtypes;
    int                  domain;
    int                  priority;
    const RadConstraint* constraints;
    int                  n_constraints;
    const RadTunable*    tunables;
    int                  n_tunables;
    const void*          reserved;
    RadInitFn            init;
    RadFiniFn            fini;
    RadLaunchFn          launch;
    RadScratchFn         scratch;
    RadLayoutFn          layout;
    RadRelayoutFn        relayout;
    RadOpdShapeFn        opd_shape;
    RadUnrelayoutFn      unrelayout;
    const char*          replaces;
} RadKernelInfo;

/* ---- what every kernel plugin exports (src/r3d_rows.cpp:16-27, :2238-2278) ---- */
uint32_t             rad_plugin_abi_version(void);
const RadPluginInfo* rad_plugin_info(void);
int                  rad_kernel_schema_count(void);
const RadOpSchema*   rad_kernel_schema_at(int i);
int                  rad_kernel_count(void);
const RadKernelInfo* rad_kernel_at(int i);

#ifdef __cplusplus
}
#endif
#endif /* RAD_ABI_H */
