/*
 * xccl-b200: API version. The Teams API level implemented is 1.0
 * (openucx/xccl src/api/xccl_version.h:20-22); XCCL_B200_* describes this library.
 */
#ifndef XCCL_B200_VERSION_H_
#define XCCL_B200_VERSION_H_

#define XCCL_VERSION_MAJOR_SHIFT 24
#define XCCL_VERSION_MINOR_SHIFT 16
#define XCCL_VERSION(major, minor) \
    (((major) << XCCL_VERSION_MAJOR_SHIFT) | ((minor) << XCCL_VERSION_MINOR_SHIFT))

#define XCCL_API_MAJOR   1
#define XCCL_API_MINOR   0
#define XCCL_API_VERSION XCCL_VERSION(XCCL_API_MAJOR, XCCL_API_MINOR)

#define XCCL_B200_VERSION_STRING "0.1.0"

#endif
