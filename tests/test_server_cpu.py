"""Bundles, the OpenAI-compatible server and cross-request batching on the CPU backend."""
import http.client
import json
import threading

import pytest

from inference_b200.bundles import RuntimeCatalog, RuntimeCatalogError, runtime_b200, runtime_cpu
from inference_b200.contracts.core_llm import LoadSpec, Message, Sampling, TextLlmRequest
from inference_b200.contracts.core_llm.prepare import SnapshotPreparerRegistryBuilder
from inference_b200.contracts.core_llm.registry import TextLlmRegistryBuilder
from inference_b200.testkit.synthetic import write_snapshot


@pytest.fixture(scope="module")
def snapshot(tmp_path_factory):
    d = tmp_path_factory.mktemp("snap")
    write_snapshot(d)
    return d


def test_catalogs_validate_and_snapshot():
    for bundle, backend, llm in ((runtime_b200, "b200", "b200-llama"), (runtime_cpu, "cpu", "cpu-llama")):
        cat = bundle.catalog()
        snap = json.loads(cat.snapshot().to_json())
        assert snap["backend"] == backend and snap["text_llm_ids"] == [llm, llm.replace("llama", "llava"), llm.replace("llama", "qwen3-vl")]
        assert snap["snapshot_preparer_backends"] == [backend] and len(snap["generator_ids"]) == 37
        assert snap["audio_backend"] == backend and snap["audio_transcriber_ids"] == ["whisper"]
        assert snap["audio_generator_ids"] == [("" if backend == "b200" else "cpu_") + n for n in ("kokoro_82m", "moss_sfx_v2", "moss_ttsd_v05", "acestep_v15_turbo", "moss_tts_realtime")]


def test_catalog_rejects_mixed_backends_and_missing_preparer():
    with pytest.raises(RuntimeCatalogError) as e:
        RuntimeCatalog.try_new("cuda", "b200", runtime_cpu.provider_registry(), runtime_cpu.text_registry(),
                               SnapshotPreparerRegistryBuilder().build())
    msg = str(e.value)
    assert "uses backend 'cpu' in the 'b200' runtime" in msg and "no snapshot preparer" in msg
    with pytest.raises(RuntimeCatalogError):
        RuntimeCatalog.try_new("", "cpu", runtime_cpu.provider_registry(), TextLlmRegistryBuilder().build(),
                               runtime_cpu.snapshot_preparer_registry())


def _post(port, body, stream=False):
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=60)
    c.request("POST", "/v1/chat/completions", json.dumps(body), {"Content-Type": "application/json"})
    r = c.getresponse()
    data = r.read()
    c.close()
    return r.status, data


def test_server_routes_and_batching(snapshot):
    from inference_b200.server import serve_in_thread

    llm = runtime_cpu.catalog().text().load_for_model(LoadSpec.dense(str(snapshot)))
    direct = llm.complete(TextLlmRequest(messages=[Message.user("w3 w4 w5")], max_new_tokens=6,
                                         sampling=Sampling.greedy()))
    httpd, service, _ = serve_in_thread(llm, "tiny", port=0)
    port = httpd.server_address[1]
    try:
        c = http.client.HTTPConnection("127.0.0.1", port, timeout=30)
        c.request("GET", "/health")
        assert json.loads(c.getresponse().read())["status"] == "ok"
        c.request("GET", "/v1/models")
        assert json.loads(c.getresponse().read())["data"][0]["id"] == "tiny"
        c.request("GET", "/nope")
        r = c.getresponse()
        r.read()
        assert r.status == 404
        c.close()
        body = {"model": "tiny", "messages": [{"role": "user", "content": "w3 w4 w5"}], "max_tokens": 6, "temperature": 0}
        status, data = _post(port, body)
        j = json.loads(data)
        assert status == 200 and j["object"] == "chat.completion"
        assert j["choices"][0]["message"]["content"] == direct.text
        assert j["usage"]["completion_tokens"] == direct.usage.generated_tokens
        # streaming: SSE chunks concatenate to the same text and end with [DONE]
        status, data = _post(port, dict(body, stream=True))
        lines = [ln[6:] for ln in data.decode().split("\n") if ln.startswith("data: ")]
        assert status == 200 and lines[-1] == "[DONE]"
        chunks = [json.loads(ln) for ln in lines[:-1]]
        text = "".join(ch["choices"][0]["delta"].get("content", "") for ch in chunks)
        assert text == direct.text and chunks[-1]["choices"][0]["finish_reason"] in ("stop", "length")
        # malformed requests
        for bad in (b"{", json.dumps({"messages": []}).encode(), json.dumps({"messages": [{"role": "x", "content": "a"}]}).encode()):
            c = http.client.HTTPConnection("127.0.0.1", port, timeout=30)
            c.request("POST", "/v1/chat/completions", bad)
            r = c.getresponse()
            assert r.status == 400 and "error" in json.loads(r.read())
            c.close()
        # concurrent clients: same answers as alone, and their decode steps were merged
        results = [None] * 6
        prompts = [f"w{3 + i} w{9 + i} w{20 + i}" for i in range(6)]
        alone = []
        for pr in prompts:
            alone.append(json.loads(_post(port, dict(body, messages=[{"role": "user", "content": pr}], max_tokens=12))[1])
                         ["choices"][0]["message"]["content"])
        before = service.batcher.stats.max_merged

        def worker(i):
            results[i] = json.loads(_post(port, dict(body, messages=[{"role": "user", "content": prompts[i]}],
                                                     max_tokens=12))[1])["choices"][0]["message"]["content"]
        ts = [threading.Thread(target=worker, args=(i,)) for i in range(6)]
        [t.start() for t in ts]
        [t.join() for t in ts]
        assert results == alone
        assert max(before, service.batcher.stats.max_merged) >= 2
        c = http.client.HTTPConnection("127.0.0.1", port, timeout=30)
        c.request("GET", "/metrics")
        m = c.getresponse().read().decode()
        assert "swb_requests_total" in m and "swb_ttft_seconds_count" in m
    finally:
        httpd.shutdown()
        httpd.server_close()
        service.close()


def test_metrics_and_tracing(tmp_path):
    from inference_b200.utils import tracing
    from inference_b200.utils.metrics import Metrics

    m = Metrics("t")
    m.inc("a")
    m.inc("a", 2)
    m.set("g", 5)
    for v in (0.002, 0.02, 0.2):
        m.observe("lat", v)
    text = m.render_prometheus()
    assert "t_a 3" in text and 't_lat_bucket{le="+Inf"} 3' in text and "t_lat_count 3" in text
    assert m.quantile("lat", 0.5) == 0.025 and m.snapshot()["gauges"]["g"] == 5
    tracing.enable(True)
    with tracing.span("outer", k=1):
        with tracing.span("inner"):
            pass
    tracing.enable(False)
    assert tracing.export_chrome_trace(str(tmp_path / "t.json")) == 2
    assert {e["name"] for e in json.load(open(tmp_path / "t.json"))["traceEvents"]} == {"outer", "inner"}
    tracing.clear()
