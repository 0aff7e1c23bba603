/* A stand-in for UCX's <ucp/api/ucp.h> for tests on machines without UCX.
 *
 * It declares, with the names, argument orders and field names of the public UCP API, exactly
 * the part that the bridge worker uses (tag-matched messages between workers that exchanged
 * their addresses), and fake_ucp.cpp beside it implements that part over Unix-domain stream
 * sockets between the processes of one host.  Nothing here comes from UCX's sources: the
 * numeric values of the constants are this file's own, which is fine because the worker is
 * compiled against whichever header it will run with.
 *
 * The stand-in reads a few environment variables so that tests can make it misbehave:
 *   FAKE_UCP_FAIL_INIT=1        ucp_init fails with UCS_ERR_NO_DEVICE
 *   FAKE_UCP_MEMORY_TYPES=...   comma list of host,cuda (default host)
 *   FAKE_UCP_VERSION=a.b.c      what ucp_get_version reports (default 1.17.0)
 */
#ifndef FAKE_UCP_API_H_
#define FAKE_UCP_API_H_

#include <stddef.h>
#include <stdint.h>

#include <ucp/api/ucp_version.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    UCS_OK = 0,
    UCS_INPROGRESS = 1,
    UCS_ERR_NO_MESSAGE = -1,
    UCS_ERR_NO_MEMORY = -4,
    UCS_ERR_INVALID_PARAM = -5,
    UCS_ERR_UNREACHABLE = -6,
    UCS_ERR_NO_DEVICE = -12,
    UCS_ERR_CANCELED = -16,
    UCS_ERR_MESSAGE_TRUNCATED = -9,
    UCS_ERR_CONNECTION_RESET = -25,
    UCS_ERR_ENDPOINT_TIMEOUT = -80,
    UCS_ERR_LAST = -100
} ucs_status_t;

typedef void* ucs_status_ptr_t;
#define UCS_PTR_IS_ERR(p)  (((uintptr_t)(p)) >= ((uintptr_t)UCS_ERR_LAST))
#define UCS_PTR_IS_PTR(p)  (((uintptr_t)(p) - 1) < ((uintptr_t)UCS_ERR_LAST - 1))
#define UCS_PTR_STATUS(p)  ((ucs_status_t)(intptr_t)(p))
#define UCS_STATUS_PTR(s)  ((void*)(intptr_t)(s))
#define UCS_BIT(i)         (1ull << (i))

typedef enum {
    UCS_MEMORY_TYPE_HOST = 0,
    UCS_MEMORY_TYPE_CUDA = 1,
    UCS_MEMORY_TYPE_CUDA_MANAGED = 2,
    UCS_MEMORY_TYPE_ROCM = 3,
    UCS_MEMORY_TYPE_UNKNOWN = 7
} ucs_memory_type_t;

typedef enum {
    UCS_THREAD_MODE_SINGLE = 0,
    UCS_THREAD_MODE_SERIALIZED = 1,
    UCS_THREAD_MODE_MULTI = 2
} ucs_thread_mode_t;

const char* ucs_status_string(ucs_status_t status);

typedef struct ucp_context* ucp_context_h;
typedef struct ucp_worker*  ucp_worker_h;
typedef struct ucp_ep*      ucp_ep_h;
typedef struct ucp_config   ucp_config_t;
typedef struct ucp_address  ucp_address_t;
typedef uint64_t            ucp_tag_t;
typedef uint64_t            ucp_datatype_t;

enum { UCP_PARAM_FIELD_FEATURES = UCS_BIT(0) };
enum { UCP_FEATURE_TAG = UCS_BIT(0) };
typedef struct ucp_params {
    uint64_t field_mask;
    uint64_t features;
} ucp_params_t;

enum { UCP_ATTR_FIELD_MEMORY_TYPES = UCS_BIT(2) };
typedef struct ucp_context_attr {
    uint64_t field_mask;
    uint64_t memory_types;
} ucp_context_attr_t;

enum { UCP_WORKER_PARAM_FIELD_THREAD_MODE = UCS_BIT(0) };
typedef struct ucp_worker_params {
    uint64_t          field_mask;
    ucs_thread_mode_t thread_mode;
} ucp_worker_params_t;

typedef enum { UCP_ERR_HANDLING_MODE_NONE = 0, UCP_ERR_HANDLING_MODE_PEER = 1 } ucp_err_handling_mode_t;
typedef void (*ucp_err_handler_cb_t)(void* arg, ucp_ep_h ep, ucs_status_t status);
typedef struct ucp_err_handler {
    ucp_err_handler_cb_t cb;
    void*                arg;
} ucp_err_handler_t;
enum {
    UCP_EP_PARAM_FIELD_REMOTE_ADDRESS    = UCS_BIT(0),
    UCP_EP_PARAM_FIELD_ERR_HANDLING_MODE = UCS_BIT(1),
    UCP_EP_PARAM_FIELD_ERR_HANDLER       = UCS_BIT(2)
};
typedef struct ucp_ep_params {
    uint64_t                field_mask;
    const ucp_address_t*    address;
    ucp_err_handling_mode_t err_mode;
    ucp_err_handler_t       err_handler;
} ucp_ep_params_t;

typedef struct ucp_tag_recv_info {
    ucp_tag_t sender_tag;
    size_t    length;
} ucp_tag_recv_info_t;

typedef void (*ucp_send_nbx_callback_t)(void* request, ucs_status_t status, void* user_data);
typedef void (*ucp_tag_recv_nbx_callback_t)(void* request, ucs_status_t status,
                                            const ucp_tag_recv_info_t* info, void* user_data);
enum {
    UCP_OP_ATTR_FIELD_CALLBACK    = UCS_BIT(1),
    UCP_OP_ATTR_FIELD_USER_DATA   = UCS_BIT(2),
    UCP_OP_ATTR_FIELD_FLAGS       = UCS_BIT(5),
    UCP_OP_ATTR_FIELD_MEMORY_TYPE = UCS_BIT(7),
    UCP_OP_ATTR_FLAG_NO_IMM_CMPL  = UCS_BIT(16)
};
enum { UCP_EP_CLOSE_FLAG_FORCE = UCS_BIT(0) };
typedef struct ucp_request_param {
    uint32_t op_attr_mask;
    uint32_t flags;
    union {
        ucp_send_nbx_callback_t     send;
        ucp_tag_recv_nbx_callback_t recv;
    } cb;
    void*             user_data;
    ucs_memory_type_t memory_type;
} ucp_request_param_t;

void ucp_get_version(unsigned* major, unsigned* minor, unsigned* release);
ucs_status_t ucp_config_read(const char* env_prefix, const char* filename, ucp_config_t** config);
void ucp_config_release(ucp_config_t* config);
ucs_status_t ucp_init(const ucp_params_t* params, const ucp_config_t* config, ucp_context_h* context);
void ucp_cleanup(ucp_context_h context);
ucs_status_t ucp_context_query(ucp_context_h context, ucp_context_attr_t* attr);
ucs_status_t ucp_worker_create(ucp_context_h context, const ucp_worker_params_t* params, ucp_worker_h* worker);
void ucp_worker_destroy(ucp_worker_h worker);
ucs_status_t ucp_worker_get_address(ucp_worker_h worker, ucp_address_t** address, size_t* length);
void ucp_worker_release_address(ucp_worker_h worker, ucp_address_t* address);
unsigned ucp_worker_progress(ucp_worker_h worker);
ucs_status_t ucp_ep_create(ucp_worker_h worker, const ucp_ep_params_t* params, ucp_ep_h* ep);
ucs_status_ptr_t ucp_ep_close_nbx(ucp_ep_h ep, const ucp_request_param_t* param);
ucs_status_ptr_t ucp_tag_send_nbx(ucp_ep_h ep, const void* buffer, size_t count, ucp_tag_t tag,
                                  const ucp_request_param_t* param);
ucs_status_ptr_t ucp_tag_recv_nbx(ucp_worker_h worker, void* buffer, size_t count, ucp_tag_t tag,
                                  ucp_tag_t tag_mask, const ucp_request_param_t* param);
ucs_status_t ucp_request_check_status(void* request);
void ucp_request_cancel(ucp_worker_h worker, void* request);
void ucp_request_free(void* request);

#ifdef __cplusplus
}
#endif
#endif
