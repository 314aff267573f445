"""Hugging Face Hub client: download (resumable, checksum-verified), search, model metadata, upload.

Endpoints and flow follow the reference's hub crate (crates/pmetal-hub/src/download.rs:62-370, search.rs:132-370,
upload.rs:111-560): files come from ``{endpoint}/{repo}/resolve/{revision}/{path}``, listings and search from
``{endpoint}/api/models``; an upload creates the repository (409 = exists), sends files of 10 MiB and more through the
git-LFS batch API (``{repo}.git/info/lfs/objects/batch`` -> PUT -> optional verify) and commits everything with one
NDJSON request (``header`` line, ``file`` lines with base64 content, ``lfsFile`` lines with the object ids).

The endpoint is ``$HF_ENDPOINT`` (default https://huggingface.co). On a machine without network every call fails with
``HubError``; ``models.loader.resolve_model_path`` keeps resolving ids through the local cache first."""
from __future__ import annotations

import base64
import hashlib
import json
import os
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Tuple

LFS_THRESHOLD = 10 * 1024 * 1024
UPLOAD_EXT = {"safetensors", "gguf", "ggml", "bin", "pt", "pth", "json", "yaml", "yml", "txt", "md", "model"}


class HubError(RuntimeError):
    pass


def endpoint() -> str:
    return os.environ.get("HF_ENDPOINT", "https://huggingface.co").rstrip("/")


def _session(token: Optional[str] = None):
    import requests
    s = requests.Session()
    s.headers["User-Agent"] = "pmetal-b200/0.1"
    if token:
        s.headers["Authorization"] = f"Bearer {token}"
    return s


def _check(resp, what: str):
    if resp.status_code >= 400:
        raise HubError(f"{what}: HTTP {resp.status_code}: {resp.text[:200]}")
    return resp


def cache_dir(repo_id: str, revision: str = "main") -> str:
    base = os.path.join(os.environ.get("HF_HOME", os.path.expanduser("~/.cache/huggingface")), "hub")
    return os.path.join(base, "models--" + repo_id.replace("/", "--"), "snapshots", revision)


def _safe_join(dest_dir: str, name: str) -> str:
    """``dest_dir/name`` for a server-supplied relative file name; raises when the result would escape ``dest_dir``."""
    if not name or os.path.isabs(name) or name.startswith(("/", "\\")):
        raise HubError(f"refusing file name {name!r}: not a relative path")
    root = os.path.abspath(dest_dir)
    path = os.path.abspath(os.path.join(root, os.path.normpath(name)))
    if os.path.commonpath([root, path]) != root or path == root:
        raise HubError(f"refusing file name {name!r}: it leaves the download directory")
    return path


def sha256_file(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as fh:
        for chunk in iter(lambda: fh.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


# ------------------------------------------------------------------------------------------------ download
def download_file(repo_id: str, filename: str, dest_dir: Optional[str] = None, revision: str = "main",
                  token: Optional[str] = None, expected_sha256: Optional[str] = None, timeout: float = 30.0,
                  expected_size: Optional[int] = None) -> str:
    """Fetch one file. A partial ``.incomplete`` file is continued with a Range request; when the server (or the caller)
    names a SHA-256, the finished file is verified and deleted on mismatch. ``filename`` is a path inside the
    repository: names that would leave ``dest_dir`` (absolute paths, ``..`` components) are rejected."""
    dest_dir = dest_dir or cache_dir(repo_id, revision)
    path = _safe_join(dest_dir, filename)
    if os.path.exists(path) and (expected_sha256 is None or sha256_file(path) == expected_sha256):
        return path
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    tmp = path + ".incomplete"
    have = os.path.getsize(tmp) if os.path.exists(tmp) else 0
    s = _session(token)
    headers = {"Range": f"bytes={have}-"} if have else {}
    url = f"{endpoint()}/{repo_id}/resolve/{revision}/{filename}"
    try:
        resp = s.get(url, headers=headers, stream=True, timeout=timeout)
    except Exception as e:
        raise HubError(f"download {url}: {e}") from e
    if resp.status_code == 416:                      # the server says nothing is left to fetch
        resp.close()
        if expected_sha256 is None and not (expected_size is not None and have == expected_size):
            # no checksum and no matching size to vouch for the partial file: fetch it again from the start
            os.remove(tmp)
            return download_file(repo_id, filename, dest_dir, revision, token, None, timeout, expected_size)
    else:
        _check(resp, f"download {filename}")
        mode = "ab" if (have and resp.status_code == 206) else "wb"
        with open(tmp, mode) as fh:
            for chunk in resp.iter_content(1 << 20):
                fh.write(chunk)
        etag = (resp.headers.get("X-Linked-Etag") or "").strip('"')
        if expected_sha256 is None and len(etag) == 64:
            expected_sha256 = etag
    if expected_sha256 is not None and sha256_file(tmp) != expected_sha256:
        os.remove(tmp)
        raise HubError(f"{filename}: checksum mismatch")
    os.replace(tmp, path)
    return path


def fetch_model_meta(repo_id: str, token: Optional[str] = None, timeout: float = 30.0) -> dict:
    try:
        resp = _session(token).get(f"{endpoint()}/api/models/{repo_id}", timeout=timeout)
    except Exception as e:
        raise HubError(f"model info {repo_id}: {e}") from e
    return _check(resp, f"model info {repo_id}").json()


MODEL_FILE_SUFFIXES = (".safetensors", ".json", ".txt", ".model", ".jinja", ".tiktoken")


def download_model(repo_id: str, revision: str = "main", token: Optional[str] = None, dest_dir: Optional[str] = None,
                   patterns: Iterable[str] = MODEL_FILE_SUFFIXES) -> str:
    """All weight, config and tokenizer files of a model repository; returns the snapshot directory."""
    meta = fetch_model_meta(repo_id, token)
    dest = dest_dir or cache_dir(repo_id, revision)
    pats = tuple(patterns)
    for sib in meta.get("siblings", []):
        name = sib.get("rfilename", "")
        if name.endswith(pats):
            size = sib.get("size") if sib.get("size") is not None else (sib.get("lfs") or {}).get("size")
            download_file(repo_id, name, dest, revision, token, (sib.get("lfs") or {}).get("sha256"),
                          expected_size=int(size) if size is not None else None)
    return dest


# ------------------------------------------------------------------------------------------------ search
@dataclass
class SearchResult:
    id: str
    downloads: int = 0
    likes: int = 0
    pipeline_tag: Optional[str] = None
    tags: List[str] = field(default_factory=list)


def search_models(query: str, limit: int = 20, tag: Optional[str] = None, token: Optional[str] = None,
                  timeout: float = 30.0) -> List[SearchResult]:
    params = {"search": query, "limit": str(limit), "sort": "downloads", "direction": "-1"}
    if tag:
        params["filter"] = tag
    try:
        resp = _session(token).get(f"{endpoint()}/api/models", params=params, timeout=timeout)
    except Exception as e:
        raise HubError(f"search: {e}") from e
    rows = _check(resp, "search").json()
    return [SearchResult(r.get("id") or r.get("modelId", ""), int(r.get("downloads") or 0), int(r.get("likes") or 0),
                         r.get("pipeline_tag"), list(r.get("tags") or [])) for r in rows]


def format_downloads(n: int) -> str:
    if n >= 1_000_000:
        return f"{n / 1e6:.1f}M"
    if n >= 1_000:
        return f"{n / 1e3:.1f}K"
    return str(n)


# ------------------------------------------------------------------------------------------------ upload
def collect_files(model_dir: str) -> List[Tuple[str, str, int]]:
    """[(local path, repo path, size)] of the uploadable files below ``model_dir``."""
    out = []
    for root, _, files in os.walk(model_dir, followlinks=True):
        for f in sorted(files):
            ext = f.rsplit(".", 1)[1] if "." in f else ""
            if ext in UPLOAD_EXT or (not ext and f in ("tokenizer", "vocab")):
                p = os.path.join(root, f)
                out.append((p, os.path.relpath(p, model_dir).replace(os.sep, "/"), os.path.getsize(p)))
    return sorted(out, key=lambda t: t[1])


def upload_model(model_dir: str, repo_id: str, token: str, private: bool = False, timeout: float = 60.0) -> dict:
    if not os.path.isdir(model_dir):
        raise ValueError(f"{model_dir!r} is not a directory")
    if "/" not in repo_id:
        raise ValueError("repo id must look like owner/name")
    org, name = repo_id.split("/", 1)
    s = _session(token)
    base = endpoint()
    try:
        r = s.post(f"{base}/api/repos/create", json={"type": "model", "name": name, "organization": org, "private": private},
                   timeout=timeout)
    except Exception as e:
        raise HubError(f"create repository: {e}") from e
    if r.status_code not in (200, 201, 409):
        raise HubError(f"create repository: HTTP {r.status_code}: {r.text[:200]}")
    files = collect_files(model_dir)
    inline = [f for f in files if f[2] < LFS_THRESHOLD]
    large = [f for f in files if f[2] >= LFS_THRESHOLD]
    lfs_entries = []
    if large:
        hashed = [(f, sha256_file(f[0])) for f in large]
        body = {"operation": "upload", "transfers": ["basic", "multipart"], "hash_algo": "sha256",
                "objects": [{"oid": oid, "size": f[2]} for f, oid in hashed]}
        hdr = {"Accept": "application/vnd.git-lfs+json", "Content-Type": "application/vnd.git-lfs+json"}
        batch = _check(s.post(f"{base}/{repo_id}.git/info/lfs/objects/batch", data=json.dumps(body), headers=hdr,
                              timeout=timeout), "LFS batch").json()
        by_oid = {oid: f for f, oid in hashed}
        for obj in batch.get("objects", []):
            f = by_oid.get(obj.get("oid"))
            if f is None:
                raise HubError(f"unknown LFS object {obj.get('oid')}")
            actions = obj.get("actions") or {}
            up = actions.get("upload")
            if up:                                    # absent when the server already has the object
                with open(f[0], "rb") as fh:
                    _check(s.put(up["href"], data=fh, headers=up.get("header") or {}, timeout=None), f"upload {f[1]}")
                ver = actions.get("verify")
                if ver:
                    _check(s.post(ver["href"], data=json.dumps({"oid": obj["oid"], "size": f[2]}),
                                  headers={**(ver.get("header") or {}), "Content-Type": "application/vnd.git-lfs+json"},
                                  timeout=timeout), f"verify {f[1]}")
        lfs_entries = [(f[1], oid, f[2]) for f, oid in hashed]
    lines = [json.dumps({"key": "header", "value": {"summary": "Upload model via pmetal",
                                                    "description": "Automated upload using the pmetal CLI"}})]
    for local, repo_path, _ in inline:
        with open(local, "rb") as fh:
            lines.append(json.dumps({"key": "file", "value": {"content": base64.b64encode(fh.read()).decode(),
                                                              "path": repo_path, "encoding": "base64"}}))
    for repo_path, oid, size in lfs_entries:
        lines.append(json.dumps({"key": "lfsFile", "value": {"path": repo_path, "algo": "sha256", "oid": oid, "size": size}}))
    _check(s.post(f"{base}/api/models/{repo_id}/commit/main", data="\n".join(lines).encode(),
                  headers={"Content-Type": "application/x-ndjson"}, timeout=timeout), "commit")
    return {"repo": repo_id, "inline_files": len(inline), "lfs_files": len(lfs_entries)}
