/* C ABI of the provider contracts (libswb200_capi.so): runtime catalog, text-LLM load / generate / stream, snapshot
 * preparation, media generator load / generate. It is the surface a non-Python host (the Rust crate in
 * bindings/rust, a C++ server) links against; behind it the framework layer is Python + PyTorch, which the library
 * embeds (or joins, when the host process already runs an interpreter).
 *
 * Conventions: every call returns 0 on success or a negative swb_status; swb_rt_last_error() gives the message of
 * the last failure on the calling thread. Structured values cross the boundary as UTF-8 JSON; strings returned
 * through `char**` are owned by the library until swb_rt_free_string(). Handles are plain integers scoped to a
 * runtime. Callbacks run on the calling thread; a non-zero return cancels the request (the contract's CancelFlag).
 */
#ifndef SWB200_CONTRACTS_H_
#define SWB200_CONTRACTS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct swb_runtime swb_runtime;

enum swb_status {
  SWB_OK = 0,
  SWB_E_INVALID = -1,     /* malformed argument / request (contract error InvalidRequest) */
  SWB_E_UNSUPPORTED = -2, /* capability gap (contract error Unsupported) */
  SWB_E_LOAD = -3,        /* weights / snapshot problem */
  SWB_E_CANCELED = -4,
  SWB_E_RUNTIME = -5,     /* any other failure inside the framework */
  SWB_E_PYTHON = -6       /* the embedded interpreter could not be started or the package not imported */
};

/* event_json: {"type":"token","id":..,"text":..,"channel":"content"|"thinking"} | {"type":"done",...} for text,
 * {"type":"step","current":..,"total":..} | {"type":"decoding"} | {"type":"loading","phase":..} for media. */
typedef int (*swb_event_cb)(const char* event_json, void* user);

/* bundle: "b200" (sm_100a kernels) or "cpu" (fp32 reference models). package_root: directory that contains the
 * `inference_b200` package, or NULL when it is importable already. */
int swb_rt_open(const char* bundle, const char* package_root, swb_runtime** out);
void swb_rt_close(swb_runtime* rt);
const char* swb_rt_last_error(void);
void swb_rt_free_string(char* s);

/* {"platform":..,"backend":..,"generator_ids":[..],"text_llm_ids":[..],"snapshot_preparer_backends":[..],...} */
int swb_rt_catalog_json(swb_runtime* rt, char** out_json);

/* load_spec_json: {"source": "<snapshot dir | gguf file>", "quantize": null|"q4"|"q8"}; provider_id NULL = select
 * by model. */
int swb_text_load(swb_runtime* rt, const char* provider_id, const char* load_spec_json, uint64_t* out_handle);
int swb_text_descriptor_json(swb_runtime* rt, uint64_t handle, char** out_json);
/* request_json: {"messages":[{"role":..,"content":..}],"max_new_tokens":..,"temperature":..,"top_p":..,"top_k":..,
 * "seed":..,"stop":[..],"json":bool}; out_json: {"text":..,"thinking":..,"finish_reason":..,"usage":{..}}. */
int swb_text_generate(swb_runtime* rt, uint64_t handle, const char* request_json, swb_event_cb on_event, void* user,
                      char** out_json);

/* spec_json: {"source":..,"out_dir":..,"quantize":null|"q4"|"q8"}; report: {"out_dir":..,"format":..,...}. */
int swb_prepare_snapshot(swb_runtime* rt, const char* spec_json, char** out_report_json);

/* load_spec_json: {"weights":"<dir>","offload_policy":"resident"|"sequential"} */
int swb_gen_load(swb_runtime* rt, const char* generator_id, const char* load_spec_json, uint64_t* out_handle);
int swb_gen_descriptor_json(swb_runtime* rt, uint64_t handle, char** out_json);
/* request_json: {"prompt":..,"width":..,"height":..,"count":..,"steps":..,"seed":..,"guidance":..,"sampler":..,
 * "scheduler":..}; out_json: {"images":[{"width":..,"height":..,"bytes":..}]}; pixels via swb_gen_image_copy. */
int swb_gen_generate(swb_runtime* rt, uint64_t handle, const char* request_json, swb_event_cb on_progress, void* user,
                     char** out_json);
/* Copies RGB8 pixels of image `index` of the handle's last generate call; returns the byte count or a status. */
long long swb_gen_image_copy(swb_runtime* rt, uint64_t handle, int index, uint8_t* dst, size_t capacity);

int swb_handle_free(swb_runtime* rt, uint64_t handle);

#ifdef __cplusplus
}
#endif
#endif /* SWB200_CONTRACTS_H_ */
