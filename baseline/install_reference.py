"""Places an unmodified copy of the reference's Python sources under ``baseline/_ref/`` (git-ignored: the copy is never
committed) so that the reference itself can be run next to this library -- its CPU search ``MCTS`` as the timed CPU
baseline, its numba.cuda ``MCTSNC`` as the GPU denominator, its ``GameRunner`` as the driver of the replay test.

    python baseline/install_reference.py [<reference root>]        (default: $MCTS_REFERENCE_ROOT, else where the reference is usually mounted)

The reference has no ``setup.py`` / ``pyproject.toml``, so there is nothing for pip to install; its modules are plain
files that import each other by name (``from mctsnc import MCTSNC``), i.e. they expect their directory on ``sys.path``.

Also writes ``baseline/_ref/gomoku/mctsnc_game_mechanics.py``: the reference switches games by editing comments in
``src/mctsnc_game_mechanics.py:59-87`` (the ``_c4`` call active, the ``_gomoku`` call commented out); this copy has the
five dispatchers switched to Gomoku and nothing else changed.  A directory holding it goes first on ``sys.path`` when
the reference's kernels are wanted for Gomoku.
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
MODULES = ["c4.py", "gomoku.py", "game_runner.py", "main.py", "mcts.py", "mctsnc.py", "mctsnc_game_mechanics.py",
           "numba_torch_compat.py", "utils.py"]
DISPATCHERS = ["is_action_legal", "take_action", "legal_actions_playout", "take_action_playout", "compute_outcome"]


def gomoku_mechanics(text):
    """The mechanics module with its five dispatchers calling the ``*_gomoku`` functions."""
    out, switched = [], 0
    for line in text.split("\n"):
        stripped = line.strip()
        for name in DISPATCHERS:
            if stripped.startswith(f"{name}_c4(") or stripped.startswith(f"return {name}_c4("):
                line = line.replace(stripped, "#" + stripped)
                switched += 1
            elif stripped.startswith(f"#{name}_gomoku(") or stripped.startswith(f"#return {name}_gomoku("):
                line = line.replace("#", "", 1)
                switched += 1
        out.append(line)
    if switched != 2 * len(DISPATCHERS):
        raise RuntimeError(f"expected {2 * len(DISPATCHERS)} dispatcher lines to switch, found {switched}")
    return "\n".join(out)


def install(reference_root):
    src = os.path.join(reference_root, "src")
    if not os.path.isdir(src):
        raise FileNotFoundError(f"{src}: reference sources not found")
    os.makedirs(os.path.join(DEST, "src"), exist_ok=True)
    os.makedirs(os.path.join(DEST, "gomoku"), exist_ok=True)
    for name in MODULES:
        shutil.copyfile(os.path.join(src, name), os.path.join(DEST, "src", name))
    with open(os.path.join(src, "mctsnc_game_mechanics.py")) as f:
        text = f.read()
    with open(os.path.join(DEST, "gomoku", "mctsnc_game_mechanics.py"), "w") as f:
        f.write(gomoku_mechanics(text))
    return DEST


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MCTS_REFERENCE_ROOT", os.path.join(os.sep, "root", "reference"))
    print(install(root))
