"""API-key management with roles, rate limits, quotas, permissions and an audit log
(easydel/workers/esurge/auth: ``EnhancedApiKeyManager``). Keys are stored hashed; the store persists to one JSON
file written atomically."""

from __future__ import annotations

import fnmatch
import hashlib
import json
import os
import secrets
import threading
import time
import typing as tp
from collections import deque
from dataclasses import asdict, dataclass, field
from enum import Enum


class ApiKeyRole(str, Enum):
    ADMIN = "admin"
    USER = "user"
    READONLY = "readonly"
    SERVICE = "service"


class ApiKeyStatus(str, Enum):
    ACTIVE = "active"
    SUSPENDED = "suspended"
    REVOKED = "revoked"
    EXPIRED = "expired"


@dataclass
class RateLimits:
    requests_per_minute: int | None = None
    requests_per_hour: int | None = None
    requests_per_day: int | None = None
    tokens_per_minute: int | None = None
    tokens_per_day: int | None = None


@dataclass
class Quota:
    max_total_tokens: int | None = None
    max_total_requests: int | None = None
    monthly_token_limit: int | None = None


@dataclass
class Permissions:
    allowed_models: list[str] | None = None
    allowed_endpoints: list[str] | None = None
    allowed_ips: list[str] | None = None
    blocked_ips: list[str] | None = None
    max_tokens_per_request: int | None = None
    enable_streaming: bool = True
    enable_function_calling: bool = True


@dataclass
class ApiKeyRecord:
    key_id: str
    key_hash: str
    key_prefix: str
    name: str
    role: str = ApiKeyRole.USER.value
    status: str = ApiKeyStatus.ACTIVE.value
    created_at: float = field(default_factory=time.time)
    expires_at: float | None = None
    last_used_at: float | None = None
    rate_limits: RateLimits = field(default_factory=RateLimits)
    quota: Quota = field(default_factory=Quota)
    permissions: Permissions = field(default_factory=Permissions)
    total_requests: int = 0
    total_prompt_tokens: int = 0
    total_completion_tokens: int = 0
    month_tokens: int = 0
    month_stamp: str = ""
    metadata: dict = field(default_factory=dict)

    def public(self) -> dict:
        d = asdict(self)
        d.pop("key_hash")
        return d


class AuthError(Exception):
    def __init__(self, message: str, status_code: int = 401):
        super().__init__(message)
        self.status_code = status_code


def _hash(key: str) -> str:
    return hashlib.sha256(key.encode()).hexdigest()


class EnhancedApiKeyManager:
    def __init__(self, require_api_key: bool = False, admin_key: str | None = None, storage_dir: str | None = None,
                 enable_persistence: bool = True, audit_limit: int = 10000):
        self.require_api_key = require_api_key
        self.admin_key_hash = _hash(admin_key) if admin_key else None
        self.path = os.path.join(storage_dir, "api_keys.json") if (storage_dir and enable_persistence) else None
        self._lock = threading.RLock()
        self._keys: dict[str, ApiKeyRecord] = {}
        self._by_hash: dict[str, str] = {}
        self._windows: dict[str, dict[str, deque]] = {}
        self.audit_log: deque = deque(maxlen=audit_limit)
        if self.path and os.path.exists(self.path):
            self._load()

    # ------------------------------------------------------------------ persistence
    def _load(self) -> None:
        with open(self.path) as f:
            raw = json.load(f)
        for d in raw.get("keys", []):
            d["rate_limits"] = RateLimits(**d.get("rate_limits", {}))
            d["quota"] = Quota(**d.get("quota", {}))
            d["permissions"] = Permissions(**d.get("permissions", {}))
            rec = ApiKeyRecord(**d)
            self._keys[rec.key_id] = rec
            self._by_hash[rec.key_hash] = rec.key_id

    def _save(self) -> None:
        if not self.path:
            return
        os.makedirs(os.path.dirname(self.path), exist_ok=True)
        tmp = self.path + ".tmp"
        with open(tmp, "w") as f:
            json.dump({"keys": [asdict(r) for r in self._keys.values()]}, f)
        os.replace(tmp, self.path)

    def _audit(self, action: str, key_id: str | None, **details) -> None:
        self.audit_log.append({"time": time.time(), "action": action, "key_id": key_id, **details})

    # ------------------------------------------------------------------ key lifecycle
    def generate_api_key(self, name: str, role: ApiKeyRole | str = ApiKeyRole.USER, expires_in_days: float | None = None,
                         rate_limits: RateLimits | None = None, quota: Quota | None = None,
                         permissions: Permissions | None = None, metadata: dict | None = None) -> tuple[str, ApiKeyRecord]:
        raw = "sk-" + secrets.token_urlsafe(32)
        rec = ApiKeyRecord(key_id="key_" + secrets.token_hex(8), key_hash=_hash(raw), key_prefix=raw[:8], name=name,
                           role=ApiKeyRole(role).value,
                           expires_at=time.time() + expires_in_days * 86400 if expires_in_days else None,
                           rate_limits=rate_limits or RateLimits(), quota=quota or Quota(),
                           permissions=permissions or Permissions(), metadata=metadata or {})
        with self._lock:
            self._keys[rec.key_id] = rec
            self._by_hash[rec.key_hash] = rec.key_id
            self._audit("create", rec.key_id, name=name, role=rec.role)
            self._save()
        return raw, rec

    def _set_status(self, key_id: str, status: ApiKeyStatus, action: str) -> bool:
        with self._lock:
            rec = self._keys.get(key_id)
            if rec is None:
                return False
            rec.status = status.value
            self._audit(action, key_id)
            self._save()
            return True

    def revoke_key(self, key_id: str) -> bool:
        return self._set_status(key_id, ApiKeyStatus.REVOKED, "revoke")

    def suspend_key(self, key_id: str) -> bool:
        return self._set_status(key_id, ApiKeyStatus.SUSPENDED, "suspend")

    def reactivate_key(self, key_id: str) -> bool:
        return self._set_status(key_id, ApiKeyStatus.ACTIVE, "reactivate")

    def delete_key(self, key_id: str) -> bool:
        with self._lock:
            rec = self._keys.pop(key_id, None)
            if rec is None:
                return False
            self._by_hash.pop(rec.key_hash, None)
            self._audit("delete", key_id)
            self._save()
            return True

    def rotate_key(self, key_id: str) -> str | None:
        with self._lock:
            rec = self._keys.get(key_id)
            if rec is None:
                return None
            self._by_hash.pop(rec.key_hash, None)
            raw = "sk-" + secrets.token_urlsafe(32)
            rec.key_hash, rec.key_prefix = _hash(raw), raw[:8]
            self._by_hash[rec.key_hash] = key_id
            self._audit("rotate", key_id)
            self._save()
            return raw

    def update_key(self, key_id: str, **fields) -> ApiKeyRecord | None:
        with self._lock:
            rec = self._keys.get(key_id)
            if rec is None:
                return None
            for k, v in fields.items():
                if k in ("rate_limits", "quota", "permissions") and isinstance(v, dict):
                    v = {"rate_limits": RateLimits, "quota": Quota, "permissions": Permissions}[k](**v)
                if hasattr(rec, k) and k not in ("key_id", "key_hash"):
                    setattr(rec, k, v)
            self._audit("update", key_id, fields=sorted(fields))
            self._save()
            return rec

    def list_keys(self, role: str | None = None, status: str | None = None) -> list[dict]:
        with self._lock:
            return [r.public() for r in self._keys.values()
                    if (role is None or r.role == role) and (status is None or r.status == status)]

    def get_key(self, key_id: str) -> ApiKeyRecord | None:
        return self._keys.get(key_id)

    # ------------------------------------------------------------------ request-time checks
    def is_admin(self, raw_key: str | None) -> bool:
        if raw_key is None:
            return False
        h = _hash(raw_key)
        if self.admin_key_hash and secrets.compare_digest(h, self.admin_key_hash):
            return True
        kid = self._by_hash.get(h)
        return kid is not None and self._keys[kid].role == ApiKeyRole.ADMIN.value and \
            self._keys[kid].status == ApiKeyStatus.ACTIVE.value

    def _window(self, key_id: str, name: str) -> deque:
        return self._windows.setdefault(key_id, {}).setdefault(name, deque())

    @staticmethod
    def _trim(q: deque, horizon: float, now: float) -> None:
        while q and q[0][0] < now - horizon:
            q.popleft()

    def authorize(self, raw_key: str | None, *, endpoint: str = "", model: str | None = None, ip: str | None = None,
                  requested_tokens: int = 0, streaming: bool = False, uses_tools: bool = False) -> ApiKeyRecord | None:
        """Raises :class:`AuthError` (401 / 403 / 429) or returns the key record (``None`` when auth is off)."""
        if raw_key is None:
            if self.require_api_key:
                raise AuthError("missing API key", 401)
            return None
        if self.admin_key_hash and secrets.compare_digest(_hash(raw_key), self.admin_key_hash):
            return None
        with self._lock:
            kid = self._by_hash.get(_hash(raw_key))
            if kid is None:
                if self.require_api_key:
                    self._audit("reject", None, reason="unknown key", ip=ip)
                    raise AuthError("invalid API key", 401)
                return None
            rec = self._keys[kid]
            now = time.time()
            if rec.expires_at and now > rec.expires_at and rec.status == ApiKeyStatus.ACTIVE.value:
                rec.status = ApiKeyStatus.EXPIRED.value
            if rec.status != ApiKeyStatus.ACTIVE.value:
                raise AuthError(f"API key is {rec.status}", 403)
            p = rec.permissions
            if p.blocked_ips and ip and any(fnmatch.fnmatch(ip, pat) for pat in p.blocked_ips):
                raise AuthError("IP address blocked", 403)
            if p.allowed_ips and ip and not any(fnmatch.fnmatch(ip, pat) for pat in p.allowed_ips):
                raise AuthError("IP address not allowed", 403)
            if p.allowed_endpoints and not any(fnmatch.fnmatch(endpoint, pat) for pat in p.allowed_endpoints):
                raise AuthError("endpoint not allowed for this key", 403)
            if p.allowed_models and model and not any(fnmatch.fnmatch(model, pat) for pat in p.allowed_models):
                raise AuthError("model not allowed for this key", 403)
            if p.max_tokens_per_request and requested_tokens > p.max_tokens_per_request:
                raise AuthError("max_tokens exceeds this key's per-request limit", 403)
            if streaming and not p.enable_streaming:
                raise AuthError("streaming is disabled for this key", 403)
            if uses_tools and not p.enable_function_calling:
                raise AuthError("function calling is disabled for this key", 403)
            if rec.role == ApiKeyRole.READONLY.value and endpoint.startswith("/v1/") and \
                    not endpoint.startswith("/v1/models"):
                raise AuthError("read-only key", 403)
            rl = rec.rate_limits
            reqs = self._window(kid, "requests")
            self._trim(reqs, 86400, now)
            for limit, horizon in ((rl.requests_per_minute, 60), (rl.requests_per_hour, 3600),
                                   (rl.requests_per_day, 86400)):
                if limit is not None and sum(1 for t, _ in reqs if t >= now - horizon) >= limit:
                    self._audit("rate_limited", kid, horizon=horizon)
                    raise AuthError("rate limit exceeded", 429)
            toks = self._window(kid, "tokens")
            self._trim(toks, 86400, now)
            for limit, horizon in ((rl.tokens_per_minute, 60), (rl.tokens_per_day, 86400)):
                if limit is not None and sum(n for t, n in toks if t >= now - horizon) >= limit:
                    raise AuthError("token rate limit exceeded", 429)
            q = rec.quota
            used = rec.total_prompt_tokens + rec.total_completion_tokens
            if q.max_total_requests is not None and rec.total_requests >= q.max_total_requests:
                raise AuthError("request quota exhausted", 429)
            if q.max_total_tokens is not None and used >= q.max_total_tokens:
                raise AuthError("token quota exhausted", 429)
            stamp = time.strftime("%Y-%m")
            if rec.month_stamp != stamp:
                rec.month_stamp, rec.month_tokens = stamp, 0
            if q.monthly_token_limit is not None and rec.month_tokens >= q.monthly_token_limit:
                raise AuthError("monthly token quota exhausted", 429)
            reqs.append((now, 1))
            rec.total_requests += 1
            rec.last_used_at = now
            return rec

    def record_usage(self, rec: ApiKeyRecord | None, prompt_tokens: int, completion_tokens: int) -> None:
        if rec is None:
            return
        with self._lock:
            rec.total_prompt_tokens += prompt_tokens
            rec.total_completion_tokens += completion_tokens
            rec.month_tokens += prompt_tokens + completion_tokens
            self._window(rec.key_id, "tokens").append((time.time(), prompt_tokens + completion_tokens))
            self._save()

    def get_audit_logs(self, limit: int = 100, key_id: str | None = None, action: str | None = None) -> list[dict]:
        rows = [r for r in self.audit_log if (key_id is None or r["key_id"] == key_id)
                and (action is None or r["action"] == action)]
        return rows[-limit:]

    def statistics(self) -> dict:
        with self._lock:
            by_status: dict[str, int] = {}
            for r in self._keys.values():
                by_status[r.status] = by_status.get(r.status, 0) + 1
            return {"total_keys": len(self._keys), "by_status": by_status,
                    "total_requests": sum(r.total_requests for r in self._keys.values()),
                    "total_tokens": sum(r.total_prompt_tokens + r.total_completion_tokens
                                        for r in self._keys.values())}
