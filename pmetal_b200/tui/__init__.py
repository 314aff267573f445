"""Terminal front end: tabbed forms over the job specifications, a job runner and a live training monitor.

Counterpart of the reference's ratatui application (crates/pmetal/src/tui/app.rs, tabs/*.rs, command_runner.rs), built
differently: every form is generated from ``core.jobs.job_specs`` (the argparse definitions), so a new sub-command or
flag shows up here without any per-tab code; jobs run as child processes of the command line and are followed through
their JSON-lines event stream; drawing is done with ``rich`` and keys are read from the terminal in raw mode."""
from .app import TuiApp, run  # noqa: F401
from .runner import Job, JobRunner  # noqa: F401
