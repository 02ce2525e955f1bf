"""FastAPI app of the dashboard.

* ``/`` one static page that polls the JSON endpoints and draws the step metrics;
* ``/api/meta`` what the run is (streams, steps seen, rollout dumps at hand), ``/api/streams``, ``/api/{stream}?since=&limit=``,
  ``/api/advisories``;
* ``/api/timeline/phases`` seconds per phase (rollout, log-probs, forward/backward, optimizer, weight update, wait) for
  every step, ``/api/timeline/bubbles`` the share of each step in which the trainer waited, ``/api/timeline/gpu`` the
  sampled GPU series per device, ``/api/timeline/engines`` the scraped engine gauges;
* ``/api/rollout/{id}/summary|groups``, ``/api/rollout/{id}/sample/{i}/tokens|messages`` the rollout inspector over the
  run's rollout dumps (``dump_reader.DumpReader``).

Reference counterpart: miles/dashboard/server.py:76-309."""
from .collector import advisories
from .store import EventStore

_PAGE = """<!doctype html><meta charset=utf-8><title>miles_b200</title>
<style>body{font:14px system-ui;margin:2em}table{border-collapse:collapse}td,th{border:1px solid #ccc;padding:2px 8px}</style>
<h1>miles_b200 run</h1><h2>Advisories</h2><ul id=adv></ul>
<h2>Tokens per second</h2><canvas id=tps width=720 height=160 style="border:1px solid #ccc"></canvas>
<h2>Last steps</h2><table id=steps></table>
<script>
async function refresh(){
  const adv = await (await fetch('api/advisories')).json();
  document.getElementById('adv').innerHTML = adv.map(a => `<li><b>${a.rule}</b>: ${a.text}</li>`).join('') || '<li>none</li>';
  const all = await (await fetch('api/metrics?limit=400')).json();
  const ys = all.map(m => +m['perf/grpo_tokens_per_s']).filter(v => isFinite(v));
  const c = document.getElementById('tps'), g = c.getContext('2d');
  g.clearRect(0, 0, c.width, c.height);
  if (ys.length > 1) {
    const hi = Math.max(...ys), lo = Math.min(...ys), sp = (hi - lo) || 1;
    g.beginPath();
    ys.forEach((v, i) => { const x = i * (c.width - 10) / (ys.length - 1) + 5, y = c.height - 5 - (v - lo) / sp * (c.height - 10); i ? g.lineTo(x, y) : g.moveTo(x, y); });
    g.stroke(); g.fillText(hi.toPrecision(4), 8, 12); g.fillText(lo.toPrecision(4), 8, c.height - 8);
  }
  const ms = all.slice(-20);
  const keys = ['step','perf/step_time','perf/rollout_time','perf/train_time','perf/grpo_tokens_per_s','train/grad_norm','rollout/reward_mean'];
  document.getElementById('steps').innerHTML = '<tr>' + keys.map(k => `<th>${k}</th>`).join('') + '</tr>' +
    ms.map(m => '<tr>' + keys.map(k => `<td>${m[k] === undefined ? '' : (+m[k]).toPrecision(5)}</td>`).join('') + '</tr>').join('');
}
refresh(); setInterval(refresh, 5000);
</script>"""


def build_dashboard_app(store: EventStore, dumps=None):
    """``dumps``: a ``dump_reader.DumpReader`` over the run's rollout dumps (None: the rollout inspector answers 404)."""
    from fastapi import FastAPI, HTTPException
    from fastapi.responses import HTMLResponse

    app = FastAPI(title="miles_b200 dashboard")

    @app.get("/", response_class=HTMLResponse)
    async def index():
        return _PAGE

    @app.get("/api/streams")
    async def streams():
        return store.streams()

    @app.get("/api/advisories")
    async def adv():
        return advisories(store)

    PHASES = ("perf/rollout_time", "perf/train_log_probs_time", "perf/train_fwd_bwd_time", "perf/train_optimizer_time",
              "perf/update_weights_time", "perf/train_wait_time", "perf/step_time")

    @app.get("/api/meta")
    async def meta():
        ms = store.tail("metrics", 1)
        return {"streams": store.streams(), "last_step": ms[-1].get("step") if ms else None,
                "rollout_dumps": dumps.rollout_ids() if dumps is not None else [], "has_tokenizer": bool(dumps and dumps.tokenizer)}

    @app.get("/api/timeline/phases")
    async def phases(limit: int = 500):
        return [{"step": m.get("step"), "t": m.get("t"), **{k.split("/", 1)[1]: m[k] for k in PHASES if k in m}}
                for m in store.tail("metrics", limit)]

    @app.get("/api/timeline/bubbles")
    async def bubbles(limit: int = 500):
        """Per step: the seconds not accounted for by rollout + training + weight update (host gaps, evaluation,
        checkpoint writes) and the share of the step the trainer spent waiting for samples."""
        out = []
        for m in store.tail("metrics", limit):
            st = m.get("perf/step_time")
            if not st:
                continue
            busy = sum(m.get(k, 0.0) for k in ("perf/rollout_time", "perf/train_time", "perf/update_weights_time"))
            out.append({"step": m.get("step"), "step_time": st, "unaccounted_s": max(st - busy, 0.0),
                        "wait_ratio": m.get("perf/wait_time_ratio", (m.get("perf/train_wait_time", 0.0)) / st)})
        return out

    @app.get("/api/timeline/gpu")
    async def gpu(since: float = 0.0, limit: int = 2000):
        series: dict = {}
        for r in list(store.read("gpus", since=since))[-limit:]:
            series.setdefault(str(r.get("gpu")), []).append({k: r.get(k) for k in ("t", "util", "mem_used", "power_w", "sm_mhz")})
        return series

    @app.get("/api/timeline/engines")
    async def engines(since: float = 0.0, limit: int = 2000):
        series: dict = {}
        for r in list(store.read("engines", since=since))[-limit:]:
            series.setdefault(r.get("engine"), []).append({k: v for k, v in r.items() if k != "engine"})
        return series

    def _or_404(v):
        if v is None:
            raise HTTPException(404, "no such rollout dump or sample (run with --save-debug-rollout-data / --dump-details)")
        return v

    @app.get("/api/rollout/{rollout_id}/summary")
    async def rollout_summary(rollout_id: int):
        return _or_404(dumps.summary(rollout_id) if dumps is not None else None)

    @app.get("/api/rollout/{rollout_id}/groups")
    async def rollout_groups(rollout_id: int):
        return _or_404(dumps.groups(rollout_id) if dumps is not None else None)

    @app.get("/api/rollout/{rollout_id}/sample/{index}/tokens")
    async def sample_tokens(rollout_id: int, index: int):
        return _or_404(dumps.sample_tokens(rollout_id, index) if dumps is not None else None)

    @app.get("/api/rollout/{rollout_id}/sample/{index}/messages")
    async def sample_messages(rollout_id: int, index: int):
        return _or_404(dumps.sample_messages(rollout_id, index) if dumps is not None else None)

    @app.get("/api/{stream}")
    async def read(stream: str, since: float = 0.0, limit: int = 200):
        recs = list(store.read(stream, since=since))
        return recs[-limit:]

    return app
