"""Generate a Prometheus + Grafana stack that scrapes the engines' /metrics endpoints (``nanoengine monitor``).
Writes docker-compose.yml, prometheus.yml and a Grafana dashboard over the `dlengine_*` metric names.
Parity: reference dlengine/monitor.py and docker/{docker-compose.monitor.yml,prometheus/,grafana/}."""
from __future__ import annotations

import json
import os
from typing import List

_PANELS = [("Throughput (tokens/s)", "dlengine_throughput_tokens_per_second"), ("Running requests", "sum(dlengine_running_requests_per_dp)"),
           ("TTFT p50 (s)", "histogram_quantile(0.5, rate(dlengine_ttft_seconds_bucket[1m]))"),
           ("TPOT p50 (s)", "histogram_quantile(0.5, rate(dlengine_tpot_seconds_bucket[1m]))"),
           ("KV blocks used", 'sum(dlengine_kv_blocks{state="used"})'), ("Prefix cache hit rate", "dlengine_prefix_cache_hit_rate"),
           ("Step latency (ms)", "dlengine_step_latency_ms"), ("Preemptions", "rate(dlengine_preemptions[1m])")]


def write_monitor_stack(out_dir: str, targets: List[str], prometheus_port: int = 9090, grafana_port: int = 3000) -> List[str]:
    os.makedirs(os.path.join(out_dir, "grafana", "dashboards"), exist_ok=True)
    os.makedirs(os.path.join(out_dir, "grafana", "provisioning", "datasources"), exist_ok=True)
    os.makedirs(os.path.join(out_dir, "grafana", "provisioning", "dashboards"), exist_ok=True)
    files = {}
    files["prometheus.yml"] = ("global:\n  scrape_interval: 2s\nscrape_configs:\n  - job_name: nanoengine\n    metrics_path: /metrics\n"
                               "    static_configs:\n      - targets: [" + ", ".join(f'"{t}"' for t in targets) + "]\n")
    files["docker-compose.yml"] = (
        "services:\n  prometheus:\n    image: prom/prometheus\n    network_mode: host\n    volumes:\n      - ./prometheus.yml:/etc/prometheus/prometheus.yml\n"
        f"    command: [\"--config.file=/etc/prometheus/prometheus.yml\", \"--web.listen-address=:{prometheus_port}\"]\n"
        "  grafana:\n    image: grafana/grafana\n    network_mode: host\n    environment:\n"
        f"      - GF_SERVER_HTTP_PORT={grafana_port}\n      - GF_AUTH_ANONYMOUS_ENABLED=true\n      - GF_AUTH_ANONYMOUS_ORG_ROLE=Admin\n"
        "    volumes:\n      - ./grafana/provisioning:/etc/grafana/provisioning\n      - ./grafana/dashboards:/var/lib/grafana/dashboards\n")
    files["grafana/provisioning/datasources/prometheus.yml"] = (
        f"apiVersion: 1\ndatasources:\n  - name: Prometheus\n    type: prometheus\n    url: http://localhost:{prometheus_port}\n    isDefault: true\n")
    files["grafana/provisioning/dashboards/default.yml"] = (
        "apiVersion: 1\nproviders:\n  - name: default\n    type: file\n    options:\n      path: /var/lib/grafana/dashboards\n")
    panels = [{"id": i + 1, "type": "timeseries", "title": t, "gridPos": {"h": 8, "w": 12, "x": 12 * (i % 2), "y": 8 * (i // 2)},
               "targets": [{"expr": e, "refId": "A"}]} for i, (t, e) in enumerate(_PANELS)]
    files["grafana/dashboards/nanoengine-overview.json"] = json.dumps({"title": "nanoengine overview", "uid": "nanoengine", "panels": panels,
                                                                       "schemaVersion": 39, "refresh": "5s", "time": {"from": "now-15m", "to": "now"}}, indent=1)
    out = []
    for rel, text in files.items():
        p = os.path.join(out_dir, rel)
        with open(p, "w") as f:
            f.write(text)
        out.append(p)
    return out
