/* Intentionally empty.
 *
 * The reference GEMM translation unit includes <arm_neon.h> unconditionally but
 * guards every NEON intrinsic with __ARM_NEON / __aarch64__.  On a non-ARM host
 * this empty header on the include path lets the reference's own portable
 * (scalar popcount) branch compile unchanged.  Test infrastructure only.
 */
