"""Python client of the batch HTTP API.

    client = BatchGenHttpClient("http://127.0.0.1:8000")
    batch = client.submit_batch("requests.jsonl", max_decoding_length=1024)     # upload + create + wait
    text = client.download_file_content(batch["output_file_id"])

Method names and behaviour follow the reference client (batchgen/batchgen_client.py; docs/client-api.md):
``upload_file``, ``create_batch``, ``get_batch``, ``wait_for_batch``, ``submit_batch``,
``download_file_content``, ``health_check``, ``close``; ``submit_inference`` raises
``LegacyInferenceDeprecated``.  503 / 429 answers with ``Retry-After`` are retried.
"""
from __future__ import annotations

import json
import os
import time
from typing import Any, Dict, List, Optional


class LegacyInferenceDeprecated(RuntimeError):
    pass


class BatchFailed(RuntimeError):
    pass


class BatchGenHttpClient:
    def __init__(self, base_url: str = "http://127.0.0.1:8000", timeout_s: float = 60.0, session=None):
        import requests
        self.base_url = base_url.rstrip("/")
        self.timeout_s = timeout_s
        self.http = session or requests.Session()

    # ------------------------------------------------------------------ plumbing
    def _request(self, method: str, path: str, retries: int = 20, **kw):
        url = self.base_url + path
        for attempt in range(retries + 1):
            r = self.http.request(method, url, timeout=self.timeout_s, **kw)
            if r.status_code in (429, 503) and attempt < retries:
                time.sleep(min(float(r.headers.get("Retry-After", "1")), 10.0))
                continue
            if r.status_code >= 400:
                raise RuntimeError(f"{method} {path} -> {r.status_code}: {r.text[:500]}")
            return r
        raise RuntimeError(f"{method} {path}: server kept answering busy")

    # ------------------------------------------------------------------ API
    def health_check(self) -> bool:
        try:
            return self.http.get(self.base_url + "/health", timeout=self.timeout_s).status_code == 200
        except Exception:  # noqa: BLE001
            return False

    def list_models(self) -> List[Dict[str, Any]]:
        return self._request("GET", "/v1/models").json()["data"]

    def upload_file(self, path_or_lines, purpose: str = "batch") -> Dict[str, Any]:
        if isinstance(path_or_lines, (list, tuple)):
            data = ("\n".join(json.dumps(l) if not isinstance(l, str) else l for l in path_or_lines) + "\n").encode()
            name = "requests.jsonl"
        else:
            with open(path_or_lines, "rb") as f:
                data = f.read()
            name = os.path.basename(path_or_lines)
        return self._request("POST", "/v1/files", files={"file": (name, data, "application/jsonl")},
                             data={"purpose": purpose}).json()

    def create_batch(self, input_file_id: str, endpoint: str = "/v1/chat/completions", completion_window: str = "24h",
                     metadata: Optional[Dict[str, str]] = None, **engine_options) -> Dict[str, Any]:
        body = {"input_file_id": input_file_id, "endpoint": endpoint, "completion_window": completion_window,
                "metadata": metadata}
        body.update({k: v for k, v in engine_options.items() if v is not None})
        return self._request("POST", "/v1/batches", json=body).json()

    def get_batch(self, batch_id: str) -> Dict[str, Any]:
        return self._request("GET", f"/v1/batches/{batch_id}").json()

    def cancel_batch(self, batch_id: str) -> Dict[str, Any]:
        return self._request("POST", f"/v1/batches/{batch_id}/cancel").json()

    def wait_for_batch(self, batch_id: str, poll_s: float = 0.5, timeout_s: Optional[float] = None,
                       raise_on_failure: bool = True) -> Dict[str, Any]:
        t0 = time.monotonic()
        while True:
            b = self.get_batch(batch_id)
            if b["status"] in ("completed", "failed", "cancelled", "expired"):
                if b["status"] == "failed" and raise_on_failure:
                    raise BatchFailed(json.dumps(b.get("errors")))
                return b
            if timeout_s is not None and time.monotonic() - t0 > timeout_s:
                raise TimeoutError(f"batch {batch_id} still {b['status']} after {timeout_s} s")
            time.sleep(poll_s)

    def submit_batch(self, path_or_lines, output_file_path: Optional[str] = None, endpoint: str = "/v1/chat/completions",
                     poll_interval: float = 0.5, timeout: Optional[float] = None, wait: bool = True,
                     **engine_options) -> Dict[str, Any]:
        """Upload, create and (unless ``wait=False``) wait for the batch; with ``output_file_path`` the output JSONL is
        saved there.  ``engine_options``: ``max_decoding_length``, ``temperature``, ``top_p``, ``top_k``, ``metadata``.
        Use ``upload_file`` + ``create_batch`` to keep several batches in flight."""
        f = self.upload_file(path_or_lines)
        batch = self.create_batch(f["id"], endpoint=endpoint, **engine_options)
        if not wait:
            return batch
        batch = self.wait_for_batch(batch["id"], poll_s=poll_interval, timeout_s=timeout)
        if output_file_path and batch.get("output_file_id"):
            with open(output_file_path, "w", encoding="utf-8") as out:
                out.write(self.download_file_content(batch["output_file_id"]))
        return batch

    def download_file_content(self, file_id: str) -> str:
        return self._request("GET", f"/v1/files/{file_id}/content").text

    def results(self, batch: Dict[str, Any]) -> List[Dict[str, Any]]:
        text = self.download_file_content(batch["output_file_id"])
        return [json.loads(l) for l in text.splitlines() if l.strip()]

    def create_session(self, metadata: Optional[Dict[str, str]] = None) -> Dict[str, Any]:
        return self._request("POST", "/v1/sessions", json={"metadata": metadata}).json()

    def turn(self, session_id: str, **body) -> Dict[str, Any]:
        return self._request("POST", "/v1/turns", json={"session_id": session_id, **body}).json()

    def close_session(self, session_id: str) -> Dict[str, Any]:
        return self._request("POST", f"/v1/sessions/{session_id}/close").json()

    def restart_workers(self) -> Dict[str, Any]:
        return self._request("POST", "/v1/workers/restart", retries=0).json()

    def workers_status(self) -> Dict[str, Any]:
        return self._request("GET", "/v1/workers/status").json()

    def submit_inference(self, *a, **kw):
        raise LegacyInferenceDeprecated("the synchronous inference API was removed; use submit_batch()")

    def close(self) -> None:
        self.http.close()
