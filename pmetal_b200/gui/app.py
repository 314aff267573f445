"""HTTP API and single-page front end over the job runner.

The reference's desktop application (crates/pmetal-gui/src-tauri/src/commands.rs: start / stop jobs, list models and
datasets, live metrics; src/routes/*: one page per job kind) is a windowed program; here the same functions are an HTTP
service any browser can open. Forms are generated in the page from ``/api/specs`` (the command-line definitions through
``core.jobs``), jobs are child processes of the command line (``tui.runner.JobRunner``), and the monitor polls
``/api/jobs/{id}`` for the metric history and the log tail. No build step, no external assets."""
from __future__ import annotations

import contextlib
import threading
from typing import Optional

from ..tui.app import FORM_TABS, scan_datasets, scan_models
from ..tui.runner import JobRunner

PAGE = """<!doctype html>
<html><head><meta charset="utf-8"><title>pmetal</title>
<style>
body{font:14px/1.4 system-ui,sans-serif;margin:0;background:#14161a;color:#e6e6e6}
nav{display:flex;flex-wrap:wrap;gap:2px;padding:6px;background:#1d2026}
nav button{background:#2a2e37;color:#ddd;border:0;padding:6px 10px;cursor:pointer}
nav button.on{background:#4b79ff;color:#fff}
main{padding:12px}
label{display:grid;grid-template-columns:260px 320px 1fr;gap:8px;margin:2px 0;align-items:center}
label small{color:#8a8f98}
input,select{background:#0f1114;color:#eee;border:1px solid #333;padding:3px}
pre{background:#0f1114;padding:8px;overflow:auto;max-height:320px}
table{border-collapse:collapse}td,th{padding:3px 10px;border-bottom:1px solid #2a2e37;text-align:left}
svg{background:#0f1114}
.run{background:#2e9d5b;color:#fff;border:0;padding:8px 18px;margin:10px 0;cursor:pointer}
</style></head><body>
<nav id="nav"></nav><main id="main"></main>
<script>
const $=(t,a={},...c)=>{const e=document.createElement(t);for(const k in a){if(k==='on')for(const ev in a.on)e.addEventListener(ev,a.on[ev]);else if(k==='text')e.textContent=a[k];else e.setAttribute(k,a[k])}c.forEach(x=>e.append(x));return e};
let specs={},tabs=[],cur='Jobs',values={},watch=null,timer=null;
async function j(u,o){const r=await fetch(u,o);const b=await r.json();if(!r.ok)throw new Error(b.detail||r.statusText);return b}
function nav(){const n=document.getElementById('nav');n.innerHTML='';for(const t of tabs)n.append($('button',{class:t===cur?'on':'',text:t,on:{click:()=>{cur=t;draw()}}}))}
function spark(v,w=520,h=90){if(!v.length)return $('span');const lo=Math.min(...v),hi=Math.max(...v),s=(hi-lo)||1;
 const p=v.map((y,i)=>`${(i/(Math.max(v.length-1,1)))*w},${h-4-(y-lo)/s*(h-8)}`).join(' ');
 const g=document.createElementNS('http://www.w3.org/2000/svg','svg');g.setAttribute('width',w);g.setAttribute('height',h);
 const l=document.createElementNS('http://www.w3.org/2000/svg','polyline');l.setAttribute('points',p);l.setAttribute('fill','none');l.setAttribute('stroke','#4b79ff');g.append(l);return g}
async function draw(){nav();clearInterval(timer);const m=document.getElementById('main');m.innerHTML='';
 if(cur==='System'){m.append($('pre',{text:JSON.stringify(await j('/api/system'),null,1)}));return}
 if(cur==='Models'||cur==='Datasets'){const rows=await j('/api/'+cur.toLowerCase());const t=$('table');
  rows.forEach(r=>t.append($('tr',{},$('td',{text:r.source||r.bytes||''}),$('td',{text:r.id||r.path}),$('td',{},$('button',{text:'use',on:{click:()=>{
   const keys=cur==='Models'?['model','student','base']:['dataset','data','input'];for(const c in specs)for(const f of specs[c].fields)if(keys.includes(f.name)&&f.kind==='string'){(values[c]=values[c]||{})[f.name]=r.id||r.path;break}}}}),
   $('button',{text:cur==='Models'?'info':'columns',on:{click:async()=>{const u=cur==='Models'?'/api/models/info?path='+encodeURIComponent(r.path||r.id):'/api/datasets/columns?path='+encodeURIComponent(r.path);
    try{det.textContent=JSON.stringify(await j(u),null,1)}catch(e){det.textContent=String(e)}}}})))));const det=$('pre');m.append(t,det);return}
 if(cur==='Jobs'){const show=async()=>{const js=await j('/api/jobs');const t=$('table',{},$('tr',{},...['id','command','state','step','loss','elapsed',''].map(h=>$('th',{text:h}))));
   js.forEach(x=>t.append($('tr',{},$('td',{text:x.id}),$('td',{text:x.command}),$('td',{text:x.state}),$('td',{text:x.metrics.step??''}),$('td',{text:x.metrics.loss?.toFixed?.(4)??''}),$('td',{text:x.elapsed.toFixed(1)+' s'}),
    $('td',{},$('button',{text:'monitor',on:{click:()=>{watch=x.id;cur='Monitor';draw()}}}),$('button',{text:'cancel',on:{click:()=>j(`/api/jobs/${x.id}/cancel`,{method:'POST'}).then(show)}})))));m.innerHTML='';m.append(t)};await show();timer=setInterval(show,1500);return}
 if(cur==='Monitor'){const show=async()=>{if(watch==null){m.textContent='no job selected';return}const x=await j('/api/jobs/'+watch);m.innerHTML='';
   m.append($('h3',{text:`job ${x.id}  ${x.command}  (${x.state})  ${x.elapsed.toFixed(1)} s`}));for(const k of ['loss','lr','tokens_per_s','grad_norm','reward'])if(x.history[k]){m.append($('div',{text:`${k}: ${x.metrics[k]}`}),spark(x.history[k]))}
   m.append($('pre',{text:x.log.join('\\n')}))};await show();timer=setInterval(show,1000);return}
 const c=tabs2cmd[cur],sp=specs[c],v=values[c]=values[c]||{};const form=$('div');
 for(const f of sp.fields){let inp;if(f.kind==='boolean'){inp=$('input',{type:'checkbox'});inp.checked=!!(v[f.name]??f.default);inp.onchange=()=>v[f.name]=inp.checked}
  else if(f.choices){inp=$('select');for(const o of f.choices)inp.append($('option',{text:o,value:o}));inp.value=v[f.name]??f.default??f.choices[0];inp.onchange=()=>v[f.name]=inp.value}
  else{inp=$('input',{value:v[f.name]??'',placeholder:f.default==null?'':String(f.default)});inp.oninput=()=>{if(inp.value==='')delete v[f.name];else v[f.name]=f.kind==='integer'?parseInt(inp.value):f.kind==='number'?parseFloat(inp.value):f.kind==='array'?inp.value.split(/\\s+/):inp.value}}
  form.append($('label',{},$('span',{text:(f.required?'* ':'')+(f.flags.at(-1)||'<'+f.name+'>')}),inp,$('small',{text:f.help||''})))}
 const out=$('pre');m.append($('h3',{text:'pmetal '+c}),form,$('button',{class:'run',text:'run',on:{click:async()=>{try{const r=await j('/api/jobs',{method:'POST',headers:{'Content-Type':'application/json'},body:JSON.stringify({command:c,values:v})});watch=r.id;cur='Monitor';draw()}catch(e){out.textContent=String(e)}}}}),out)}
let tabs2cmd={};
(async()=>{const s=await j('/api/specs');specs=s.specs;tabs2cmd=s.tabs;tabs=['System','Models','Datasets',...Object.keys(s.tabs),'Monitor','Jobs'];draw()})();
</script></body></html>"""


def create_app(runner: Optional[JobRunner] = None, model_roots=None, dataset_roots=None, settings_path: Optional[str] = None):
    from fastapi import FastAPI, HTTPException
    from fastapi.responses import HTMLResponse

    from ..core.jobs import job_specs
    runner = runner or JobRunner()
    specs = job_specs()
    lock = threading.Lock()

    @contextlib.asynccontextmanager
    async def lifespan(_app):
        yield
        runner.shutdown()                  # running jobs end with the service

    app = FastAPI(title="pmetal", lifespan=lifespan)
    app.state.runner = runner

    def job_view(j, detail: bool = False) -> dict:
        d = {"id": j.job_id, "command": j.command, "argv": j.argv, "state": j.state, "returncode": j.returncode,
             "elapsed": round(j.elapsed(), 2), "metrics": dict(j.metrics)}
        if detail:
            d["history"] = {k: v[-2000:] for k, v in j.history.items()}
            d["log"] = j.tail(60)
        return d

    def find(job_id: int):
        for j in runner.jobs:
            if j.job_id == job_id:
                return j
        raise HTTPException(404, f"no job {job_id}")

    @app.get("/", response_class=HTMLResponse)
    def page():
        return PAGE

    @app.get("/api/specs")
    def api_specs():
        tabs = {title: cmd for title, cmd in FORM_TABS if cmd in specs}
        out = {}
        for cmd in tabs.values():
            sp = specs[cmd]
            out[cmd] = {"help": sp.help, "schema": sp.json_schema(),
                        "fields": [{"name": f.name, "flags": f.flags, "kind": f.kind, "default": f.default, "required": f.required,
                                    "choices": f.choices, "help": f.help} for f in sp.fields if f.name not in ("func", "what")]}
        return {"tabs": tabs, "specs": out}

    @app.get("/api/system")
    def api_system():
        from ..utils.sysinfo import system_info
        try:
            return system_info()
        except Exception as e:
            return {"error": str(e)}

    @app.get("/api/models")
    def api_models():
        return scan_models(model_roots)

    @app.get("/api/datasets")
    def api_datasets():
        return scan_datasets(dataset_roots)

    @app.post("/api/jobs")
    def start(body: dict):
        cmd = body.get("command")
        if cmd not in specs:
            raise HTTPException(400, f"unknown command {cmd!r}")
        try:
            argv = specs[cmd].to_argv({k: v for k, v in (body.get("values") or {}).items() if v is not None})
        except ValueError as e:
            raise HTTPException(422, str(e)) from None
        with lock:
            j = runner.start(cmd, argv)
        return job_view(j)

    @app.get("/api/jobs")
    def jobs():
        with lock:
            runner.poll()
            return [job_view(j) for j in runner.jobs]

    @app.get("/api/jobs/{job_id}")
    def job(job_id: int):
        with lock:
            runner.poll()
            return job_view(find(job_id), detail=True)

    @app.post("/api/jobs/{job_id}/cancel")
    def cancel(job_id: int):
        with lock:
            j = find(job_id)
            runner.cancel(j)
            return job_view(j)

    import os

    from .library import Settings, register
    register(app, runner, Settings(settings_path or os.path.join(runner.workdir, "settings.json")), model_roots, dataset_roots)
    return app


def serve_gui(host: str = "127.0.0.1", port: int = 8090, workdir: Optional[str] = None) -> int:
    import uvicorn
    import os
    settings = os.path.join(os.path.expanduser(os.environ.get("PMETAL_CONFIG_DIR", "~/.config/pmetal")), "gui.json")
    uvicorn.run(create_app(JobRunner(workdir=workdir), settings_path=settings), host=host, port=port, log_level="info")
    return 0
