"""Python end of the contracts C ABI (csrc/capi/capi.cpp): one entry point, `dispatch(runtime_id, op, payload_json)`,
returning "<status>\\n<body>". Structured values are JSON; callbacks are C function pointers invoked through ctypes
on the calling thread (a non-zero return trips the request's CancelFlag)."""
from __future__ import annotations

import ctypes
import itertools
import json
import threading

from .contracts.errors import Canceled, InferenceError, InvalidRequest, LoadError, Unsupported

OK, E_INVALID, E_UNSUPPORTED, E_LOAD, E_CANCELED, E_RUNTIME = 0, -1, -2, -3, -4, -5
_EVENT_CB = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_char_p, ctypes.c_void_p)
_lock = threading.Lock()
_ids = itertools.count(1)
_runtimes: dict[int, "_Runtime"] = {}


class _Runtime:
    def __init__(self, bundle: str):
        from .bundles import runtime_b200, runtime_cpu

        mods = {"b200": runtime_b200, "cpu": runtime_cpu}
        if bundle not in mods:
            raise InvalidRequest(f"unknown bundle {bundle!r} (known: {sorted(mods)})")
        self.catalog = mods[bundle].catalog()
        self.handles: dict[int, object] = {}
        self.images: dict[int, list] = {}
        self.next = itertools.count(1)

    def put(self, obj) -> int:
        h = next(self.next)
        self.handles[h] = obj
        return h

    def get(self, h: int):
        if h not in self.handles:
            raise InvalidRequest(f"unknown handle {h}")
        return self.handles[h]


def _emitter(cb_addr: int, user: int, cancel):
    if not cb_addr:
        return lambda obj: None
    fn = _EVENT_CB(cb_addr)

    def emit(obj: dict) -> None:
        if fn(json.dumps(obj).encode(), user or None):
            cancel.cancel()
    return emit


def _descriptor_json(d) -> dict:
    import dataclasses
    import enum

    def enc(v):
        if dataclasses.is_dataclass(v):
            return {k: enc(x) for k, x in dataclasses.asdict(v).items()}
        if isinstance(v, enum.Enum):
            return v.value
        if isinstance(v, (list, tuple)):
            return [enc(x) for x in v]
        if isinstance(v, dict):
            return {k: enc(x) for k, x in v.items()}
        return v
    return enc(d)


def _text_request(j: dict):
    from .contracts.core_llm import Constraint, Message, Role, Sampling, TextLlmRequest

    roles = {"system": Role.SYSTEM, "user": Role.USER, "assistant": Role.ASSISTANT, "tool": Role.TOOL}
    msgs = []
    for m in j.get("messages", []):
        if m.get("role") not in roles:
            raise InvalidRequest(f"unknown role {m.get('role')!r}")
        msgs.append(Message.text(roles[m["role"]], str(m.get("content", ""))))
    temp = float(j.get("temperature", 0.0))
    sampling = Sampling.greedy() if temp <= 0 else Sampling(temperature=temp, top_p=float(j.get("top_p", 1.0)),
                                                            top_k=int(j.get("top_k", 0)))
    return TextLlmRequest(messages=msgs, max_new_tokens=int(j.get("max_new_tokens", 128)), sampling=sampling,
                          seed=j.get("seed"), stop=list(j.get("stop", [])),
                          constraint=Constraint.JSON if j.get("json") else None)


def _op(rt: _Runtime | None, op: str, p: dict):
    if op == "open":
        r = _Runtime(p.get("bundle", "b200"))
        with _lock:
            rid = next(_ids)
            _runtimes[rid] = r
        return str(rid)
    if rt is None:
        raise InvalidRequest("runtime is not open")
    if op == "close":
        return ""
    if op == "catalog":
        return rt.catalog.snapshot().to_json()
    if op == "text_load":
        from .contracts.core_llm import LoadSpec, Quantize

        s = p["spec"]
        spec = LoadSpec(s["source"], {"q4": Quantize.Q4, "q8": Quantize.Q8, None: None}[s.get("quantize")])
        reg = rt.catalog.text()
        llm = reg.load_textllm(p["provider_id"], spec) if p.get("provider_id") else reg.load_for_model(spec)
        return str(rt.put(llm))
    if op == "descriptor":
        return json.dumps(_descriptor_json(rt.get(p["handle"]).descriptor()))
    if op == "text_generate":
        from .contracts.core_llm.output import DoneEvent, TokenEvent

        llm = rt.get(p["handle"])
        req = _text_request(p["request"])
        emit = _emitter(p.get("callback", 0), p.get("user", 0), req.cancel)

        def on_event(ev):
            if isinstance(ev, TokenEvent):
                emit({"type": "token", "id": ev.id, "text": ev.text, "index": ev.index, "channel": ev.channel.value})
            elif isinstance(ev, DoneEvent):
                emit({"type": "done", "finish_reason": ev.finish_reason.value,
                      "prompt_tokens": ev.usage.prompt_tokens, "generated_tokens": ev.usage.generated_tokens})
        out = llm.generate(req, on_event)
        return json.dumps({"text": out.text, "thinking": out.thinking,
                           "finish_reason": out.finish_reason.value if out.finish_reason else None,
                           "usage": {"prompt_tokens": out.usage.prompt_tokens,
                                     "generated_tokens": out.usage.generated_tokens}})
    if op == "prepare":
        from .contracts.core_llm import Quantize
        from .contracts.core_llm.prepare import PrepareSpec

        s = p["spec"]
        q = {"q4": Quantize.Q4, "q8": Quantize.Q8, None: None}[s.get("quantize")]
        spec = PrepareSpec.dense(s["source"], s["out_dir"]) if q is None else PrepareSpec.quantized(s["source"],
                                                                                                   s["out_dir"], q)
        rep = rt.catalog.preparers().prepare_snapshot(spec)
        return json.dumps(_descriptor_json(rep), default=str)
    if op == "gen_load":
        from .contracts.gen_core import LoadSpec, OffloadPolicy, WeightsSource

        s = p["spec"]
        spec = LoadSpec(weights=WeightsSource.dir(s["weights"]),
                        offload_policy=OffloadPolicy(s.get("offload_policy", "resident")))
        return str(rt.put(rt.catalog.media().load(p["id"], spec)))
    if op == "gen_generate":
        from .contracts.gen_core import GenerationRequest, ProgressDecoding, ProgressLoading, ProgressStep

        g = rt.get(p["handle"])
        fields = {k: v for k, v in p["request"].items()
                  if k in ("prompt", "width", "height", "count", "steps", "seed", "guidance", "true_cfg", "sampler", "scheduler",
                           "scheduler_shift", "negative_prompt", "frames", "fps")}
        req = GenerationRequest(**fields)
        emit = _emitter(p.get("callback", 0), p.get("user", 0), req.cancel)

        def on_progress(ev):
            if isinstance(ev, ProgressStep):
                emit({"type": "step", "current": ev.current, "total": ev.total})
            elif isinstance(ev, ProgressDecoding):
                emit({"type": "decoding"})
            elif isinstance(ev, ProgressLoading):
                emit({"type": "loading", "phase": ev.phase.value})
        out = g.generate(req, on_progress)
        pictures = out.images or out.video_frames            # a video's frames are fetched like images, by index
        rt.images[p["handle"]] = pictures
        return json.dumps({"kind": out.kind, "fps": out.fps,
                           "images": [{"width": i.width, "height": i.height, "bytes": len(i.pixels)} for i in pictures]})
    if op == "gen_image_copy":
        imgs = rt.images.get(p["handle"], [])
        if not 0 <= p["index"] < len(imgs):
            raise InvalidRequest(f"image index {p['index']} out of range (have {len(imgs)})")
        px = imgs[p["index"]].pixels
        if p["capacity"] < len(px):
            raise InvalidRequest(f"buffer of {p['capacity']} bytes is smaller than the image ({len(px)} bytes)")
        ctypes.memmove(p["dst"], px, len(px))
        return str(len(px))
    if op == "free":
        rt.handles.pop(p["handle"], None)
        rt.images.pop(p["handle"], None)
        return ""
    raise InvalidRequest(f"unknown operation {op!r}")


def dispatch(runtime_id: int, op: str, payload_json: str) -> str:
    try:
        payload = json.loads(payload_json) if payload_json else {}
        rt = _runtimes.get(runtime_id)
        body = _op(rt, op, payload)
        if op == "close":
            with _lock:
                _runtimes.pop(runtime_id, None)
        return f"{OK}\n{body}"
    except Canceled as e:
        return f"{E_CANCELED}\n{e}"
    except Unsupported as e:
        return f"{E_UNSUPPORTED}\n{e}"
    except LoadError as e:
        return f"{E_LOAD}\n{e}"
    except (InvalidRequest, KeyError, ValueError, json.JSONDecodeError) as e:
        return f"{E_INVALID}\n{type(e).__name__}: {e}"
    except InferenceError as e:
        return f"{E_RUNTIME}\n{e}"
    except Exception as e:   # nothing may propagate into the C caller
        return f"{E_RUNTIME}\n{type(e).__name__}: {e}"
