"""The contracts C ABI (libswb200_capi.so) driven through its exported symbols on the CPU bundle."""
import ctypes
import json

import pytest

from inference_b200._native.build import build_capi
from inference_b200.media.flux import write_synthetic_snapshot
from inference_b200.testkit.synthetic import write_snapshot

CB = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_char_p, ctypes.c_void_p)


@pytest.fixture(scope="module")
def lib():
    L = ctypes.CDLL(str(build_capi()))
    L.swb_rt_last_error.restype = ctypes.c_char_p
    L.swb_gen_image_copy.restype = ctypes.c_longlong
    L.swb_gen_image_copy.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t]
    for name in ("swb_text_generate", "swb_gen_generate"):
        getattr(L, name).argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_char_p, CB, ctypes.c_void_p,
                                     ctypes.POINTER(ctypes.c_char_p)]
    L.swb_rt_open.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]
    L.swb_rt_catalog_json.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_char_p)]
    L.swb_text_load.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_char_p, ctypes.POINTER(ctypes.c_uint64)]
    L.swb_gen_load.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_char_p, ctypes.POINTER(ctypes.c_uint64)]
    L.swb_text_descriptor_json.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.POINTER(ctypes.c_char_p)]
    L.swb_handle_free.argtypes = [ctypes.c_void_p, ctypes.c_uint64]
    L.swb_rt_close.argtypes = [ctypes.c_void_p]
    return L


def _take(L, p):
    s = ctypes.cast(p, ctypes.c_char_p).value.decode()
    return s


def test_text_and_media_through_the_c_abi(lib, tmp_path):
    snap = tmp_path / "llm"
    write_snapshot(snap)
    flux = write_synthetic_snapshot(tmp_path / "flux")
    rt = ctypes.c_void_p()
    assert lib.swb_rt_open(b"nope", None, ctypes.byref(rt)) == -1 and b"unknown bundle" in lib.swb_rt_last_error()
    assert lib.swb_rt_open(b"cpu", None, ctypes.byref(rt)) == 0
    out = ctypes.c_char_p()
    assert lib.swb_rt_catalog_json(rt, ctypes.byref(out)) == 0
    cat = json.loads(out.value)
    assert cat["backend"] == "cpu" and cat["text_llm_ids"] == ["cpu-llama", "cpu-llava", "cpu-qwen3-vl"]
    # ---- text ------------------------------------------------------------------------------------------
    h = ctypes.c_uint64()
    assert lib.swb_text_load(rt, None, json.dumps({"source": str(tmp_path / "missing")}).encode(), ctypes.byref(h)) < 0
    assert lib.swb_text_load(rt, None, json.dumps({"source": str(snap)}).encode(), ctypes.byref(h)) == 0
    assert lib.swb_text_descriptor_json(rt, h, ctypes.byref(out)) == 0
    assert json.loads(out.value)["backend"] == "cpu"
    events = []

    @CB
    def on_event(js, user):
        events.append(json.loads(js))
        return 0
    req = {"messages": [{"role": "user", "content": "w3 w4 w5"}], "max_new_tokens": 5}
    assert lib.swb_text_generate(rt, h, json.dumps(req).encode(), on_event, None, ctypes.byref(out)) == 0
    res = json.loads(out.value)
    toks = [e for e in events if e["type"] == "token"]
    assert events[-1]["type"] == "done" and "".join(t["text"] for t in toks) == res["text"]
    assert res["usage"]["generated_tokens"] <= 5
    # a callback that returns non-zero cancels the request
    seen = []

    @CB
    def cancel_after_first(js, user):
        seen.append(js)
        return 1
    rc = lib.swb_text_generate(rt, h, json.dumps(dict(req, max_new_tokens=50)).encode(), cancel_after_first, None,
                               ctypes.byref(out))
    assert rc in (0, -4) and len(seen) <= 3
    assert lib.swb_text_generate(rt, h, b'{"messages": [{"role": "martian", "content": "x"}]}', CB(0), None,
                                 ctypes.byref(out)) == -1
    assert lib.swb_handle_free(rt, h) == 0
    assert lib.swb_text_descriptor_json(rt, h, ctypes.byref(out)) == -1
    # ---- media -----------------------------------------------------------------------------------------
    g = ctypes.c_uint64()
    assert lib.swb_gen_load(rt, b"cpu_flux1_dev", json.dumps({"weights": str(flux)}).encode(), ctypes.byref(g)) == 0
    prog = []

    @CB
    def on_progress(js, user):
        prog.append(json.loads(js)["type"])
        return 0
    greq = {"prompt": "a fox", "width": 256, "height": 256, "steps": 2, "seed": 1}
    assert lib.swb_gen_generate(rt, g, json.dumps(greq).encode(), on_progress, None, ctypes.byref(out)) == 0
    meta = json.loads(out.value)["images"][0]
    assert meta == {"width": 256, "height": 256, "bytes": 256 * 256 * 3}
    assert prog.count("step") == 2 and prog.count("decoding") == 1
    buf = (ctypes.c_uint8 * meta["bytes"])()
    assert lib.swb_gen_image_copy(rt, g, 0, buf, meta["bytes"]) == meta["bytes"]
    assert lib.swb_gen_image_copy(rt, g, 0, buf, 10) == -1 and lib.swb_gen_image_copy(rt, g, 3, buf, meta["bytes"]) == -1
    assert lib.swb_gen_generate(rt, g, json.dumps(dict(greq, width=250)).encode(), CB(0), None, ctypes.byref(out)) < 0
    # a video generator: the frames come back through the same image-copy call
    from inference_b200.media.wan import write_synthetic_snapshot as write_wan

    wan = write_wan(tmp_path / "wan")
    v = ctypes.c_uint64()
    assert lib.swb_gen_load(rt, b"cpu_wan2_2_t2v_14b", json.dumps({"weights": str(wan)}).encode(), ctypes.byref(v)) == 0
    vreq = {"prompt": "a fox runs", "width": 256, "height": 256, "steps": 2, "seed": 1, "frames": 5, "fps": 12}
    assert lib.swb_gen_generate(rt, v, json.dumps(vreq).encode(), CB(0), None, ctypes.byref(out)) == 0
    vmeta = json.loads(out.value)
    assert vmeta["kind"] == "video" and vmeta["fps"] == 12 and len(vmeta["images"]) == 5
    assert lib.swb_gen_image_copy(rt, v, 4, buf, meta["bytes"]) == meta["bytes"]
    lib.swb_rt_close(rt)


def test_standalone_c_host_embeds_an_interpreter(tmp_path):
    """A plain C program (no Python in the process) links the library, which opens libpython and starts one."""
    import os
    import shutil
    import site
    import subprocess
    from pathlib import Path

    repo = Path(__file__).resolve().parent.parent
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    libdir = build_capi().parent
    exe = tmp_path / "c_host"
    subprocess.run([cc, "-o", str(exe), str(repo / "examples" / "c_host.c"), "-I",
                    str(repo / "inference_b200" / "csrc" / "include"), "-L", str(libdir), "-lswb200_capi",
                    f"-Wl,-rpath,{libdir}"], check=True)
    env = dict(os.environ, PYTHONPATH=os.pathsep.join(site.getsitepackages()))
    r = subprocess.run([str(exe), str(repo)], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout + r.stderr
    assert '"text_llm_ids": ["cpu-llama", "cpu-llava", "cpu-qwen3-vl"]' in r.stdout
