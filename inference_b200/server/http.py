"""OpenAI-compatible HTTP front end over any `TextLlm` (role of mlx-llm-server's main.rs:170-470, with two
differences: connections are served concurrently, and their decode steps are merged by `BatchingBackend` when the
provider exposes a decode backend).

Routes: POST /v1/chat/completions (JSON, or SSE when `stream` is true), GET /v1/models, GET /health, GET /metrics.
Deadlines: 10 s to read a request, 10 min per response; a failed socket write trips the request's CancelFlag so the
generation loop stops at its next token."""
from __future__ import annotations

import json
import threading
import time
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

from ..contracts.core_llm.output import DoneEvent, TokenEvent
from ..contracts.errors import Canceled, InferenceError, InvalidRequest, Unsupported
from ..utils import logging as log
from ..utils.metrics import Metrics
from . import openai

READ_TIMEOUT_S = 10.0
MAX_BODY_BYTES = 8 << 20


class LlmService:
    """What the handlers need: the model, its public id, metrics, and (optionally) the batching proxy."""

    def __init__(self, llm, model_id: str, batching: bool = True, max_batch: int = 64):
        self.llm, self.model_id, self.metrics = llm, model_id, Metrics()
        self.batcher = None
        inner = getattr(llm, "backend", None)
        if batching and inner is not None and hasattr(inner, "forward_greedy"):
            from ..engine.batching import BatchingBackend

            self.batcher = BatchingBackend(inner, max_batch=max_batch)
            llm.backend = self.batcher
        self.started = time.time()

    def close(self) -> None:
        if self.batcher is not None:
            self.llm.backend = self.batcher.inner
            self.batcher.close()

    def generate(self, req, on_event):
        if self.batcher is None:
            return self.llm.generate(req, on_event)
        with self.batcher:
            return self.llm.generate(req, on_event)


def make_handler(service: LlmService):
    class Handler(BaseHTTPRequestHandler):
        protocol_version = "HTTP/1.1"
        server_version = "inference-b200"

        def log_message(self, fmt, *args):   # route access logs through the structured logger
            log.debug("http", line=fmt % args)

        def setup(self):
            super().setup()
            self.connection.settimeout(READ_TIMEOUT_S)

        # ---- helpers ---------------------------------------------------------------------------------------
        def _json(self, code: int, body: dict) -> None:
            data = json.dumps(body).encode()
            self.send_response(code)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)

        def _error(self, code: int, message: str, kind: str = "invalid_request_error") -> None:
            service.metrics.inc("http_errors_total")
            self._json(code, openai.error_body(message, kind))

        # ---- routes ------------------------------------------------------------------------------------------
        def do_GET(self):
            if self.path == "/health":
                self._json(200, {"status": "ok", "model": service.model_id, "uptime_s": round(time.time() - service.started, 1)})
            elif self.path == "/v1/models":
                self._json(200, {"object": "list", "data": [{"id": service.model_id, "object": "model",
                                                              "owned_by": "inference-b200"}]})
            elif self.path == "/metrics":
                if service.batcher is not None:
                    st = service.batcher.stats
                    service.metrics.set("batch_steps", st.steps)
                    service.metrics.set("batch_rows", st.rows)
                    service.metrics.set("batch_max_merged", st.max_merged)
                data = service.metrics.render_prometheus().encode()
                self.send_response(200)
                self.send_header("Content-Type", "text/plain; version=0.0.4")
                self.send_header("Content-Length", str(len(data)))
                self.end_headers()
                self.wfile.write(data)
            else:
                self._error(404, f"no route for GET {self.path}", "not_found")

        def do_POST(self):
            if self.path != "/v1/chat/completions":
                return self._error(404, f"no route for POST {self.path}", "not_found")
            try:
                n = int(self.headers.get("Content-Length", "0"))
            except ValueError:
                return self._error(400, "bad Content-Length")
            if n <= 0 or n > MAX_BODY_BYTES:
                return self._error(413 if n > MAX_BODY_BYTES else 400, "request body missing or too large")
            body = self.rfile.read(n)
            try:
                req, stream, _model = openai.parse_chat_request(body)
                service.llm.validate(req)
            except Unsupported as e:
                return self._error(400, str(e), "unsupported")
            except (InvalidRequest, InferenceError) as e:
                return self._error(400, str(e))
            except Exception as e:  # noqa: BLE001  (a malformed field that slipped past validation: still a 400)
                return self._error(400, f"malformed request: {type(e).__name__}: {e}")
            service.metrics.inc("requests_total")
            service.metrics.add_gauge("requests_in_flight", 1)
            t0 = time.perf_counter()
            try:
                (self._stream if stream else self._complete)(req, t0)
            finally:
                service.metrics.add_gauge("requests_in_flight", -1)
                service.metrics.observe("request_seconds", time.perf_counter() - t0)

        def _complete(self, req, t0):
            first = [None]

            def on_event(ev):
                if isinstance(ev, TokenEvent) and first[0] is None:
                    first[0] = time.perf_counter() - t0
            try:
                out = service.generate(req, on_event)
            except Canceled:
                return self._error(499, "request cancelled", "cancelled")
            except InferenceError as e:
                return self._error(500, str(e), "server_error")
            except Exception as e:  # noqa: BLE001  (a device / runtime failure must still produce a response)
                service.metrics.inc("request_errors_total")
                return self._error(500, f"{type(e).__name__}: {e}", "server_error")
            if first[0] is not None:
                service.metrics.observe("ttft_seconds", first[0])
            service.metrics.inc("generated_tokens_total", out.usage.generated_tokens)
            service.metrics.inc("prompt_tokens_total", out.usage.prompt_tokens)
            self._json(200, openai.completion_body(openai.completion_id(), service.model_id, out))

        def _stream(self, req, t0):
            cid = openai.completion_id()
            self.send_response(200)
            self.send_header("Content-Type", "text/event-stream")
            self.send_header("Cache-Control", "no-cache")
            self.send_header("Connection", "close")
            self.end_headers()
            self.close_connection = True
            state = {"first": True}

            def send(obj) -> None:
                try:
                    self.wfile.write(b"data: " + (obj if isinstance(obj, bytes) else json.dumps(obj).encode()) + b"\n\n")
                    self.wfile.flush()
                except OSError:
                    req.cancel.cancel()        # the client went away: stop generating

            def on_event(ev):
                if isinstance(ev, TokenEvent) and state["first"]:
                    service.metrics.observe("ttft_seconds", time.perf_counter() - t0)
                chunk = openai.chunk_body(cid, service.model_id, ev, state["first"])
                if chunk is not None:
                    send(chunk)
                    state["first"] = False
                if isinstance(ev, DoneEvent):
                    service.metrics.inc("generated_tokens_total", ev.usage.generated_tokens)
                    service.metrics.inc("prompt_tokens_total", ev.usage.prompt_tokens)
            try:
                service.generate(req, on_event)
            except Canceled:
                pass
            except InferenceError as e:
                send(openai.error_body(str(e), "server_error"))
            except Exception as e:  # noqa: BLE001
                service.metrics.inc("request_errors_total")
                send(openai.error_body(f"{type(e).__name__}: {e}", "server_error"))
            send(b"[DONE]")

    return Handler


def serve(llm, model_id: str, host: str = "127.0.0.1", port: int = 8000, batching: bool = True,
          max_batch: int = 64) -> tuple[ThreadingHTTPServer, LlmService]:
    """Bind and return (server, service); call server.serve_forever() (or run it in a thread) to accept."""
    service = LlmService(llm, model_id, batching=batching, max_batch=max_batch)
    httpd = ThreadingHTTPServer((host, port), make_handler(service))
    httpd.daemon_threads = True
    log.info("server_listening", host=host, port=httpd.server_address[1], model=model_id, batching=batching)
    return httpd, service


def serve_in_thread(llm, model_id: str, **kw):
    httpd, service = serve(llm, model_id, **kw)
    t = threading.Thread(target=httpd.serve_forever, name="swb-http", daemon=True)
    t.start()
    return httpd, service, t
