"""Hub client against an in-process fake of the hub's HTTP API (no network)."""
import base64
import hashlib
import json
import threading
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

import pytest

from pmetal_b200 import hub

BLOB = bytes(range(256)) * 4096               # 1 MiB
BIG = b"x" * (hub.LFS_THRESHOLD + 5)


class Fake(BaseHTTPRequestHandler):
    log = []
    store = {}

    def log_message(self, *a):
        pass

    def _json(self, obj, code=200, headers=None):
        raw = json.dumps(obj).encode()
        self.send_response(code)
        self.send_header("Content-Type", "application/json")
        self.send_header("Content-Length", str(len(raw)))
        for k, v in (headers or {}).items():
            self.send_header(k, v)
        self.end_headers()
        self.wfile.write(raw)

    def do_GET(self):
        Fake.log.append(("GET", self.path, dict(self.headers)))
        if self.path.startswith("/api/models?"):
            return self._json([{"id": "org/tiny", "downloads": 1234567, "likes": 3, "pipeline_tag": "text-generation", "tags": ["a"]}])
        if self.path == "/api/models/org/tiny":
            return self._json({"id": "org/tiny", "siblings": [
                {"rfilename": "config.json"}, {"rfilename": "model.safetensors", "lfs": {"sha256": hashlib.sha256(BLOB).hexdigest()}},
                {"rfilename": "notes.pdf"}]})
        if self.path == "/org/tiny/resolve/main/config.json":
            raw = b'{"model_type": "llama"}'
        elif self.path == "/org/tiny/resolve/main/model.safetensors":
            raw = BLOB
        elif self.path == "/org/tiny/resolve/main/bad.bin":
            raw = b"corrupt"
        else:
            return self._json({"error": "not found"}, 404)
        start = 0
        rng = self.headers.get("Range")
        if rng:
            start = int(rng.split("=")[1].split("-")[0])
            if start >= len(raw):
                self.send_response(416)
                self.send_header("Content-Length", "0")
                self.end_headers()
                return
            self.send_response(206)
        else:
            self.send_response(200)
        body = raw[start:]
        self.send_header("Content-Length", str(len(body)))
        if self.path.endswith("bad.bin"):
            self.send_header("X-Linked-Etag", '"' + "0" * 64 + '"')
        self.end_headers()
        self.wfile.write(body)

    def _body(self):
        return self.rfile.read(int(self.headers.get("Content-Length", 0)))

    def do_POST(self):
        body = self._body()
        Fake.log.append(("POST", self.path, body))
        host = f"http://127.0.0.1:{self.server.server_port}"
        if self.path == "/api/repos/create":
            return self._json({"url": "x"}, 409)
        if self.path.endswith("/info/lfs/objects/batch"):
            req = json.loads(body)
            objs = [{"oid": o["oid"], "size": o["size"], "actions": {
                "upload": {"href": f"{host}/lfs/{o['oid']}", "header": {"X-Up": "1"}},
                "verify": {"href": f"{host}/verify/{o['oid']}"}}} for o in req["objects"]]
            return self._json({"objects": objs})
        if self.path.startswith("/verify/"):
            ok = json.loads(body)["oid"] in Fake.store
            return self._json({}, 200 if ok else 404)
        if self.path == "/api/models/me/up/commit/main":
            return self._json({"commitUrl": "c"})
        return self._json({"error": "?"}, 404)

    def do_PUT(self):
        body = self._body()
        Fake.log.append(("PUT", self.path, len(body), self.headers.get("X-Up")))
        Fake.store[self.path.rsplit("/", 1)[1]] = hashlib.sha256(body).hexdigest()
        self._json({})


@pytest.fixture()
def server(monkeypatch, tmp_path):
    srv = ThreadingHTTPServer(("127.0.0.1", 0), Fake)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    Fake.log.clear()
    Fake.store.clear()
    monkeypatch.setenv("HF_ENDPOINT", f"http://127.0.0.1:{srv.server_port}")
    monkeypatch.setenv("HF_HOME", str(tmp_path / "hf"))
    yield srv
    srv.shutdown()


def test_search_download_resume_and_checksum(server, tmp_path):
    res = hub.search_models("tiny", limit=5, tag="text-generation", token="tok")
    assert res[0].id == "org/tiny" and hub.format_downloads(res[0].downloads) == "1.2M" and hub.format_downloads(999) == "999"
    get = [e for e in Fake.log if e[0] == "GET"][0]
    assert "search=tiny" in get[1] and "filter=text-generation" in get[1] and get[2]["Authorization"] == "Bearer tok"
    d = hub.download_model("org/tiny")
    assert d.endswith("models--org--tiny/snapshots/main")
    assert open(f"{d}/model.safetensors", "rb").read() == BLOB and json.load(open(f"{d}/config.json"))["model_type"] == "llama"
    assert not (tmp_path / "hf" / "hub" / "models--org--tiny" / "snapshots" / "main" / "notes.pdf").exists()
    # resume: a partial file is continued with a Range request and verified
    dest = tmp_path / "resume"
    dest.mkdir()
    (dest / "model.safetensors.incomplete").write_bytes(BLOB[:300000])
    Fake.log.clear()
    p = hub.download_file("org/tiny", "model.safetensors", str(dest), expected_sha256=hashlib.sha256(BLOB).hexdigest())
    assert open(p, "rb").read() == BLOB
    assert [e for e in Fake.log if e[0] == "GET"][0][2]["Range"] == "bytes=300000-"
    with pytest.raises(hub.HubError, match="checksum"):
        hub.download_file("org/tiny", "bad.bin", str(dest))
    assert not (dest / "bad.bin").exists() and not (dest / "bad.bin.incomplete").exists()
    with pytest.raises(hub.HubError, match="404"):
        hub.download_file("org/tiny", "missing.json", str(dest))


def test_download_rejects_names_that_leave_the_directory(server, tmp_path):
    dest = tmp_path / "snap"
    dest.mkdir()
    for bad in ("../escape.json", "/etc/passwd", "a/../../b.json", ""):
        with pytest.raises(hub.HubError, match="refusing"):
            hub.download_file("org/tiny", bad, str(dest))
    assert not (tmp_path / "escape.json").exists()
    assert not any(e[0] == "GET" for e in Fake.log)           # nothing was requested for a refused name
    p = hub.download_file("org/tiny", "config.json", str(dest))
    assert p == str(dest / "config.json")


def test_range_not_satisfiable_without_checksum_is_not_trusted(server, tmp_path):
    dest = tmp_path / "r416"
    dest.mkdir()
    # a stale partial file that is as long as the real one but holds other bytes; no checksum is known
    (dest / "config.json.incomplete").write_bytes(b"X" * len(b'{"model_type": "llama"}'))
    p = hub.download_file("org/tiny", "config.json", str(dest))
    assert json.load(open(p))["model_type"] == "llama"
    # with a matching size on record the finished partial file is accepted as is
    (dest / "again.incomplete").write_bytes(b"x")
    (dest / "config.json").unlink()
    (dest / "config.json.incomplete").write_bytes(b'{"model_type": "llama"}')
    p = hub.download_file("org/tiny", "config.json", str(dest), expected_size=len(b'{"model_type": "llama"}'))
    assert json.load(open(p))["model_type"] == "llama"


def test_upload_splits_inline_and_lfs_files(server, tmp_path):
    m = tmp_path / "model"
    (m / "sub").mkdir(parents=True)
    (m / "config.json").write_text('{"a": 1}')
    (m / "sub" / "notes.md").write_text("hi")
    (m / "model.safetensors").write_bytes(BIG)
    (m / "skip.exe").write_bytes(b"no")
    rep = hub.upload_model(str(m), "me/up", "secret")
    assert rep == {"repo": "me/up", "inline_files": 2, "lfs_files": 1}
    oid = hashlib.sha256(BIG).hexdigest()
    put = [e for e in Fake.log if e[0] == "PUT"][0]
    assert put[1] == f"/lfs/{oid}" and put[2] == len(BIG) and put[3] == "1" and Fake.store[oid] == oid
    commit = [e for e in Fake.log if e[0] == "POST" and e[1].endswith("/commit/main")][0][2].decode().split("\n")
    rows = [json.loads(x) for x in commit]
    assert rows[0]["key"] == "header" and [r["key"] for r in rows[1:]] == ["file", "file", "lfsFile"]
    assert rows[1]["value"]["path"] == "config.json" and base64.b64decode(rows[1]["value"]["content"]) == b'{"a": 1}'
    assert rows[2]["value"]["path"] == "sub/notes.md"
    assert rows[3]["value"] == {"path": "model.safetensors", "algo": "sha256", "oid": oid, "size": len(BIG)}
    with pytest.raises(ValueError):
        hub.upload_model(str(m), "noslash", "t")


def test_offline_errors_are_hub_errors(monkeypatch):
    monkeypatch.setenv("HF_ENDPOINT", "http://127.0.0.1:9")            # nothing listens there
    with pytest.raises(hub.HubError):
        hub.search_models("x", timeout=2)
    with pytest.raises(hub.HubError):
        hub.fetch_model_meta("a/b", timeout=2)
