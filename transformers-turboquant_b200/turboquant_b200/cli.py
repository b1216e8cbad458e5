"""Command-line entry of the package (reference: src/transformers_turboquant/cli.py:1-21, one `validate` command).

    python -m turboquant_b200.cli validate [--contexts ...] [--bits ...] [--layers N]
"""

from __future__ import annotations

import typer

app = typer.Typer(help="HuggingFace integration for TurboQuant KV compression (B200 kernels).")


@app.command(context_settings={"allow_extra_args": True, "ignore_unknown_options": True})
def validate(ctx: typer.Context) -> None:
    """Estimator-quality validation on a Qwen2.5-3B-shaped random-init model (requires a GPU)."""
    from .validate import main
    main(list(ctx.args))


@app.callback()
def _root() -> None:
    """Keeps `validate` a sub-command, as in the reference's CLI, although it is the only one."""


if __name__ == "__main__":
    app()
