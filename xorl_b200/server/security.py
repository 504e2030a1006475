"""Boundaries of the training server: names that become path components, paths that must stay
below a root, and outbound HTTP endpoints (inference engines registered for weight sync).

Same guarantees as the reference's helpers (src/xorl/server/security.py): identifiers are a short
alphanumeric alphabet, artifact paths are resolved and confined to the server's output root with
symlinked components refused, and an endpoint is parsed, optionally checked against the allow-list
``XORL_OUTBOUND_ENDPOINT_ALLOWLIST`` (hostnames, addresses, CIDR blocks, comma separated), resolved
once, rejected when it points at link-local / multicast / unspecified / reserved space, and
returned as an address literal so that a second DNS answer cannot redirect the request.
"""
from __future__ import annotations

import ipaddress
import os
import re
import socket
from pathlib import Path
from typing import List, Optional, Tuple, Union

ALLOWLIST_ENV = "XORL_OUTBOUND_ENDPOINT_ALLOWLIST"
ARTIFACT_ROOT_ENV = "XORL_SERVER_ARTIFACT_ROOT"
_ID = re.compile(r"[A-Za-z0-9][A-Za-z0-9_.-]{0,127}")
_LABEL = r"[A-Za-z0-9](?:[A-Za-z0-9-]{0,61}[A-Za-z0-9])?"
_HOST = re.compile(rf"(?=.{{1,253}}\.?$){_LABEL}(?:\.{_LABEL})*\.?")
PathLike = Union[str, os.PathLike]


def validate_identifier(value, name: str = "identifier") -> str:
    text = str(value)
    if not _ID.fullmatch(text) or set(text) <= {"."}:
        raise ValueError(f"{name} must start with a letter or digit and use only letters, digits, '_', '-', '.' "
                         f"(at most 128 characters): {text!r}")
    return text


def confine_path(root: PathLike, candidate: PathLike, *, must_exist: bool = False,
                 reject_symlinks: bool = True) -> Path:
    """``candidate`` (relative to ``root`` unless absolute) resolved, and required to lie below ``root``."""
    base = Path(root).expanduser().resolve()
    raw = Path(candidate).expanduser()
    target = raw if raw.is_absolute() else base / raw
    if reject_symlinks:
        node = target
        while node != base and node != node.parent:
            if node.is_symlink():
                raise ValueError(f"symlinked path component refused: {node}")
            node = node.parent
    resolved = target.resolve(strict=False)
    if resolved != base and base not in resolved.parents:
        raise ValueError(f"path {candidate!s} leaves the configured root {base}")
    if must_exist and not resolved.exists():
        raise FileNotFoundError(str(resolved))
    return resolved


def artifact_path(candidate: PathLike, root: Optional[PathLike] = None, must_exist: bool = False) -> Path:
    """A checkpoint / export path of the server below its artifact root (argument, else
    ``XORL_SERVER_ARTIFACT_ROOT``, else ``./checkpoints``)."""
    if candidate is None or not str(candidate).strip():
        raise ValueError("artifact path must not be empty")
    if root is None:
        root = os.environ.get(ARTIFACT_ROOT_ENV, "").strip() or Path.cwd() / "checkpoints"
    return confine_path(root, candidate, must_exist=must_exist)


def _allowlist() -> List[str]:
    return [e.strip() for e in os.environ.get(ALLOWLIST_ENV, "").split(",") if e.strip()]


def _in_networks(addr, entries: List[str]) -> bool:
    for e in entries:
        try:
            if addr in ipaddress.ip_network(e, strict=False):
                return True
        except ValueError:
            pass
    return False


def validate_endpoint(host: str, port, *, require_allowlist: bool = False) -> Tuple[str, int]:
    """(address literal, port) of a safe outbound endpoint, or ValueError."""
    h = str(host).strip().rstrip(".")
    if not h or any(c in h for c in "/\\@?#\0\r\n "):
        raise ValueError(f"invalid endpoint host {host!r}")
    try:
        p = int(port)
    except (TypeError, ValueError):
        raise ValueError(f"invalid endpoint port {port!r}") from None
    if not 1 <= p <= 65535:
        raise ValueError(f"endpoint port {p} outside [1, 65535]")
    entries = _allowlist()
    named = any("/" not in e and e.rstrip(".").lower() == h.lower() for e in entries)
    try:
        addrs = [ipaddress.ip_address(h.strip("[]"))]
        literal = True
    except ValueError:
        literal = False
        if not _HOST.fullmatch(h):
            raise ValueError(f"invalid endpoint hostname {h!r}") from None
        try:
            infos = socket.getaddrinfo(h, p, type=socket.SOCK_STREAM)
        except socket.gaierror:
            raise ValueError(f"endpoint hostname {h!r} does not resolve") from None
        addrs = [ipaddress.ip_address(i[4][0]) for i in infos if i[0] in (socket.AF_INET, socket.AF_INET6)]
        if not addrs:
            raise ValueError(f"endpoint hostname {h!r} has no IP address")
    if require_allowlist:
        if not entries:
            if h.lower() != "localhost" and not all(a.is_loopback for a in addrs):
                raise ValueError(f"endpoint {h!r} is not allowed: set {ALLOWLIST_ENV}")
        elif not named and not (literal and _in_networks(addrs[0], entries)):
            raise ValueError(f"endpoint {h!r} is not in {ALLOWLIST_ENV}")
    for a in addrs:
        unsafe = a.is_link_local or _is_group_address(a) or a.is_unspecified or (a.is_reserved and not a.is_loopback)
        if unsafe and not _in_networks(a, entries):
            raise ValueError(f"unsafe endpoint address {a}")
        if require_allowlist and a.is_private and not (a.is_loopback or named or _in_networks(a, entries)):
            raise ValueError(f"private endpoint address {a} needs an entry in {ALLOWLIST_ENV}")
    return str(addrs[0]), p


_GROUP_NETWORKS = (ipaddress.ip_network("224.0.0.0/4"), ipaddress.ip_network("ff00::/8"))


def _is_group_address(a) -> bool:
    """One-to-many (group) addresses: 224.0.0.0/4 and ff00::/8."""
    return any(a.version == n.version and a in n for n in _GROUP_NETWORKS)


def endpoint_url(host: str, port, path: str, *, require_allowlist: bool = False) -> str:
    if not path.startswith("/") or any(c in path for c in "\0\r\n?#"):
        raise ValueError(f"invalid endpoint path {path!r}")
    a, p = validate_endpoint(host, port, require_allowlist=require_allowlist)
    return f"http://[{a}]:{p}{path}" if ":" in a else f"http://{a}:{p}{path}"
