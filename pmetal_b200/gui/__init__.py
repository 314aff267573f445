"""Browser front end: the job forms, runner and monitor of the terminal application behind a small HTTP API and one
static page (counterpart of the reference's desktop application, crates/pmetal-gui: Tauri commands + Svelte routes)."""
from .app import create_app, serve_gui  # noqa: F401
