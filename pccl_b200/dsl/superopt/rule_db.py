"""On-disk cache of discovered rules and device profiles.

Files live under ``~/.pccl/superopt/`` (``rules_k{k}.json`` per pattern size,
``profiles/{name}.json`` per calibrated device) — the same location and file
names as the reference so caches are interchangeable (reference:
pccl/dsl/superopt/rule_db.py:11-68).
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Dict, List, Optional

from .rule import RewriteRule


def _cache_dir() -> Path:
    return Path.home() / ".pccl" / "superopt"


def _profiles_dir() -> Path:
    return _cache_dir() / "profiles"


def _rules_path(k: int) -> Path:
    return _cache_dir() / f"rules_k{k}.json"


def _ensure_dirs() -> None:
    _profiles_dir().mkdir(parents=True, exist_ok=True)


def save_rules(k: int, rules: List[RewriteRule]) -> Path:
    _ensure_dirs()
    path = _rules_path(k)
    path.write_text(json.dumps([rule.to_dict() for rule in rules], indent=2))
    return path


def load_rules(k: int) -> List[RewriteRule]:
    path = _rules_path(k)
    if not path.exists():
        return []
    return [RewriteRule.from_dict(entry) for entry in json.loads(path.read_text())]


def load_all_rules(max_k: int = 6) -> List[RewriteRule]:
    return [rule for k in range(1, max_k + 1) for rule in load_rules(k)]


def clear_rules(k: Optional[int] = None) -> None:
    targets = [_rules_path(k)] if k is not None else list(_cache_dir().glob("rules_k*.json"))
    for path in targets:
        if path.exists():
            path.unlink()


def save_profile(name: str, profile: Dict[str, Any]) -> Path:
    _ensure_dirs()
    path = _profiles_dir() / f"{name}.json"
    path.write_text(json.dumps(profile, indent=2))
    return path


def load_profile(name: str) -> Optional[Dict[str, Any]]:
    path = _profiles_dir() / f"{name}.json"
    return json.loads(path.read_text()) if path.exists() else None
