"""File-backed LRU store of Responses-API conversations (easydel/workers/response_store): ``previous_response_id``
lookups return the message history that produced a response so that the next turn can be appended."""

from __future__ import annotations

import json
import os
import threading
from collections import OrderedDict


class ResponseStore:
    def __init__(self, directory: str | None = None, max_items: int = 4096):
        self.dir, self.max_items = directory, max_items
        self._mem: OrderedDict[str, dict] = OrderedDict()
        self._lock = threading.Lock()
        if directory:
            os.makedirs(directory, exist_ok=True)
            files = sorted((os.path.getmtime(os.path.join(directory, f)), f) for f in os.listdir(directory)
                           if f.endswith(".json"))
            for _, f in files[-max_items:]:
                self._mem[f[:-5]] = None          # loaded lazily

    def _path(self, rid: str) -> str:
        return os.path.join(self.dir, rid + ".json")

    def put(self, response_id: str, record: dict) -> None:
        with self._lock:
            self._mem[response_id] = record
            self._mem.move_to_end(response_id)
            if self.dir:
                tmp = self._path(response_id) + ".tmp"
                with open(tmp, "w") as f:
                    json.dump(record, f)
                os.replace(tmp, self._path(response_id))
            while len(self._mem) > self.max_items:
                old, _ = self._mem.popitem(last=False)
                if self.dir and os.path.exists(self._path(old)):
                    os.remove(self._path(old))

    def get(self, response_id: str) -> dict | None:
        with self._lock:
            if response_id not in self._mem:
                return None
            rec = self._mem[response_id]
            if rec is None and self.dir:
                with open(self._path(response_id)) as f:
                    rec = json.load(f)
                self._mem[response_id] = rec
            self._mem.move_to_end(response_id)
            return rec

    def delete(self, response_id: str) -> bool:
        with self._lock:
            found = self._mem.pop(response_id, "missing") != "missing"
            if self.dir and os.path.exists(self._path(response_id)):
                os.remove(self._path(response_id))
            return found

    def __len__(self) -> int:
        return len(self._mem)
