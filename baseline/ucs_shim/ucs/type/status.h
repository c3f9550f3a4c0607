#ifndef UCS_SHIM_STATUS_H_
#define UCS_SHIM_STATUS_H_
typedef enum { UCS_OK = 0, UCS_INPROGRESS = 1, UCS_ERR_NO_MEMORY = -4, UCS_ERR_INVALID_PARAM = -5, UCS_ERR_NO_ELEM = -12 } ucs_status_t;
#endif
