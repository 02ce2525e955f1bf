"""FastAPI app of the dashboard: ``/api/streams``, ``/api/{stream}?since=&limit=``, ``/api/advisories`` and ``/`` (one
static page that polls the JSON endpoints and draws the step metrics as tables)."""
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


def build_dashboard_app(store: EventStore):
    from fastapi import FastAPI
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

    @app.get("/api/{stream}")
    async def read(stream: str, since: float = 0.0, limit: int = 200):
        recs = list(store.read(stream, since=since))
        return recs[-limit:]

    return app
