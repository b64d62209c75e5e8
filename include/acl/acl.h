/*
 * acl/acl.h - source-compatibility shim.
 *
 * The reference's public header includes the Ascend runtime header of this name for one type, `aclrtStream`
 * (include/cann_ops_tensor.h:20, :196).  On B200 a stream is a CUDA stream; the type is kept as an opaque pointer
 * so that this header needs no CUDA include and client code keeps compiling unchanged.
 */
#ifndef OPS_TENSOR_B200_ACL_SHIM_H
#define OPS_TENSOR_B200_ACL_SHIM_H

typedef void* aclrtStream; /* holds a cudaStream_t */

#endif
