"""Model directory cache and (optional) download from the Hugging Face hub.

Cache layout and markers follow the reference fetcher (safetensors/.../fetch/ModelFetcher.java:19-47,60,170): models live in
``~/.deliverance/<owner>_<name>/`` (override with ``DELIVERANCE_HOME``), a finished download carries ``.finished``, the
token comes from ``HF_TOKEN`` (or the ``huggingface.auth.token`` property of the reference = ``HUGGINGFACE_AUTH_TOKEN`` here),
files are listed through ``/api/models/<id>`` and fetched from ``/resolve/main/<file>``. Without network access
``maybe_download`` fails with a clear error unless the directory is already complete.
"""
from __future__ import annotations

import json
import os
import shutil
import urllib.request
from typing import Callable, Optional

FINISHED = ".finished"
DEFAULT_PATTERNS = (".safetensors", ".json", ".model", ".txt", ".jinja")


class ModelFetcher:
    def __init__(self, owner: str, name: str, home: Optional[str] = None, endpoint: str = "https://huggingface.co",
                 opener: Optional[Callable[[str, dict], bytes]] = None):
        self.owner, self.name = owner, name
        self.home = os.path.expanduser(home or os.environ.get("DELIVERANCE_HOME", "~/.deliverance"))
        self.endpoint = endpoint.rstrip("/")
        self._open = opener or self._http_get

    @staticmethod
    def from_id(model_id: str, **kw) -> "ModelFetcher":
        owner, _, name = model_id.partition("/")
        if not name:
            raise ValueError("model id must look like 'owner/name'")
        return ModelFetcher(owner, name, **kw)

    @property
    def model_dir(self) -> str:
        return os.path.join(self.home, f"{self.owner}_{self.name}")

    def is_complete(self) -> bool:
        return os.path.exists(os.path.join(self.model_dir, FINISHED))

    def token(self) -> Optional[str]:
        return os.environ.get("HF_TOKEN") or os.environ.get("HUGGINGFACE_AUTH_TOKEN")

    def _http_get(self, url: str, headers: dict) -> bytes:
        req = urllib.request.Request(url, headers=headers)
        with urllib.request.urlopen(req, timeout=60) as r:
            return r.read()

    def list_files(self) -> list[str]:
        hdr = {"Authorization": f"Bearer {self.token()}"} if self.token() else {}
        meta = json.loads(self._open(f"{self.endpoint}/api/models/{self.owner}/{self.name}", hdr))
        return [s["rfilename"] for s in meta.get("siblings", [])]

    def maybe_download(self, patterns=DEFAULT_PATTERNS) -> str:
        """Return the local directory, downloading what is missing. A directory with ``.finished`` is used as is."""
        if self.is_complete():
            return self.model_dir
        staging = self.model_dir + ".partial"
        os.makedirs(staging, exist_ok=True)
        hdr = {"Authorization": f"Bearer {self.token()}"} if self.token() else {}
        try:
            files = [f for f in self.list_files() if f.endswith(tuple(patterns))]
            for f in files:
                dst = os.path.join(staging, f)
                if os.path.exists(dst):
                    continue
                os.makedirs(os.path.dirname(dst) or staging, exist_ok=True)
                data = self._open(f"{self.endpoint}/{self.owner}/{self.name}/resolve/main/{f}", hdr)
                with open(dst + ".tmp", "wb") as fh:
                    fh.write(data)
                os.replace(dst + ".tmp", dst)
        except OSError as e:
            raise RuntimeError(f"cannot download {self.owner}/{self.name} (offline?): {e}; place the model under {self.model_dir} "
                               f"and create {FINISHED}") from e
        with open(os.path.join(staging, FINISHED), "w") as fh:
            fh.write("ok\n")
        if os.path.exists(self.model_dir):
            shutil.rmtree(self.model_dir)
        os.replace(staging, self.model_dir)
        return self.model_dir
