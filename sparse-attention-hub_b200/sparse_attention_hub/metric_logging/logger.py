"""Process-wide micro-metric logger (reference: sparse_attention_hub/metric_logging/logger.py).

Kept small: metrics are registered by name and type, switched on explicitly,
buffered in a bounded deque and flushed as JSON lines.  The research-attention
path logs `research_attention_density` and `research_attention_output_error`
through it when they are enabled.
"""

import json
import os
import time
from collections import deque
from dataclasses import asdict, dataclass, field
from typing import Any, Deque, Dict, List, Optional, Union


@dataclass
class LogEvent:
    timestamp: float
    metric: str
    value: Any
    metadata: Dict[str, Any] = field(default_factory=dict)
    location: str = ""


class MicroMetricLogger:
    """Singleton; `MicroMetricLogger()` always returns the same object."""

    _instance: Optional["MicroMetricLogger"] = None
    _registered_metrics: Dict[str, type] = {}

    def __new__(cls, *args: Any, **kwargs: Any) -> "MicroMetricLogger":
        if cls._instance is None:
            cls._instance = super().__new__(cls)
            cls._instance._initialised = False
        return cls._instance

    def __init__(self, log_path: Optional[str] = None, flush_every: int = 1000,
                 enabled_metrics: Union[List[str], str, None] = None,
                 max_records: Optional[int] = None, sampling_factor: float = 1.0) -> None:
        if not self._initialised:
            self.log_path: Optional[str] = None
            self.flush_every = flush_every
            self.max_records = max_records
            self.sampling_factor = sampling_factor
            self.enabled_metrics: set = set()
            self.log_queue: Deque[LogEvent] = deque(maxlen=10000)
            self._total = 0
            self._initialised = True
        if log_path is not None:
            self.log_path = log_path
            os.makedirs(log_path, exist_ok=True)
        if enabled_metrics is not None:
            self.enable_metrics(enabled_metrics)

    @classmethod
    def register_metric(cls, identifier: str, dtype: type) -> None:
        cls._registered_metrics[identifier] = dtype

    @classmethod
    def get_registered_metrics(cls) -> Dict[str, type]:
        return cls._registered_metrics.copy()

    def enable_metrics(self, metrics: Union[List[str], str, None] = None) -> None:
        if metrics == "all":
            self.enabled_metrics = set(self._registered_metrics)
        elif isinstance(metrics, (list, set, tuple)):
            self.enabled_metrics = {m for m in metrics if m in self._registered_metrics}
        else:
            self.enabled_metrics = set()

    def is_metric_enabled(self, identifier: str) -> bool:
        return identifier in self.enabled_metrics

    def is_logging_configured(self) -> bool:
        return self.log_path is not None

    def log(self, identifier: str, value: Any, metadata: Optional[Dict[str, Any]] = None) -> None:
        if identifier not in self.enabled_metrics or self.log_path is None:
            return
        if self.max_records is not None and self._total >= self.max_records:
            return
        self._total += 1
        self.log_queue.append(LogEvent(time.time(), identifier, value, metadata or {}))
        if len(self.log_queue) >= self.flush_every:
            self.flush()

    def flush(self) -> None:
        if self.log_path is None or not self.log_queue:
            return
        with open(os.path.join(self.log_path, "micro_metrics.jsonl"), "a", encoding="utf-8") as f:
            while self.log_queue:
                f.write(json.dumps(asdict(self.log_queue.popleft())) + "\n")
