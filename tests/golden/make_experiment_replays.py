"""Turns experiment archives of the reference (its ``experiments/*.zip``: the matches its authors ran on their GPU, with
the step count, chosen move and statistics of every search) into a compact fixture for replay tests.

    python tests/golden/make_experiment_replays.py <reference root> [games per experiment]

For every selected match-up the fixture keeps the MCTSNC settings, the moves of the first games, and per MCTSNC search
(in the order they were run: one instance plays all games of a match, its random streams run on from search to search)
the recorded steps, best action, n_root, win flag, n, n_wins, playouts, max depth, max size, mean size and mean depth.
The reference replays such archives itself (``src/main.py`` with REPRODUCE_EXPERIMENT, ``src/game_runner.py:86-92``).
"""
import glob
import json
import os
import re
import sys
import zipfile

import numpy as np

SELECTED = [
    "mcts_5_inf_vanilla;mctsnc_1_inf_1_32_ocp_thrifty", "mcts_5_inf_vanilla;mctsnc_1_inf_1_32_ocp_prodigal",
    "mcts_5_inf_vanilla;mctsnc_1_inf_1_32_acp_thrifty", "mcts_5_inf_vanilla;mctsnc_1_inf_1_32_acp_prodigal",
    "mcts_5_inf_vanilla;mctsnc_1_inf_2_64_ocp_thrifty", "mcts_5_inf_vanilla;mctsnc_1_inf_4_128_acp_thrifty",
    "mcts_5_inf_vanilla;mctsnc_1_inf_8_256_ocp_prodigal", "mcts_5_inf_vanilla;mctsnc_1_inf_4_256_acp_prodigal",
    "mcts_5_inf_vanilla;mctsnc_5_inf_4_256_acp_prodigal", "mctsnc_5_inf_4_256_acp_thrifty;mctsnc_5_inf_4_256_acp_prodigal",
    "mcts_5_inf_vanilla;mctsnc_1_inf_8_256_acp_thrifty", "mcts_5_inf_vanilla;mctsnc_1_inf_8_32_acp_prodigal",
    "mcts_5_inf_vanilla;mctsnc_1_inf_2_256_ocp_prodigal", "mcts_5_inf_vanilla;mctsnc_1_inf_4_64_ocp_thrifty",
    "mcts_5_inf_vanilla;mctsnc_1_inf_1_256_acp_thrifty", "mcts_5_inf_vanilla;mctsnc_1_inf_8_128_ocp_thrifty",
    "mcts_5_inf_vanilla;mctsnc_1_inf_2_128_acp_prodigal", "mctsnc_5_inf_4_128_ocp_thrifty;mctsnc_5_inf_4_256_ocp_prodigal",
]
INSTANCE = re.compile(r"MCTSNC\(search_time_limit=([\d.]+), search_steps_limit=(\w+), n_trees=(\d+), n_playouts=(\d+), "
                      r"variant='(\w+)', device_memory=([\d.]+), ucb_c=([\d.]+), seed: (\d+)\)")


def extract(path, n_games):
    z = zipfile.ZipFile(path)
    d = json.loads(z.read([n for n in z.namelist() if n.endswith(".json")][0]))
    info = d["matchup_info"]
    out = {"ai_a": info["ai_a_instance"], "ai_b": info["ai_b_instance"], "games": []}
    for g in range(1, n_games + 1):
        game = d["games_infos"][str(g)]
        moves, searches = [], []
        for r in range(1, len(game["moves_rounds"]) + 1):
            rnd = game["moves_rounds"][str(r)]
            for colour in ("black", "white"):
                if colour + "_best_action_info" not in rnd:
                    continue
                best, perf = rnd[colour + "_best_action_info"], rnd[colour + "_performance_info"]
                moves.append(int(best["index"]))
                if "trees" in perf:   # an MCTSNC search
                    t = perf["trees"]
                    searches.append([len(moves) - 1, int(perf["steps"]), int(best["index"]), int(best["n_root"]),
                                     int(bool(best["win_flag"])), int(best["n"]), int(best["n_wins"]), int(perf["playouts"]),
                                     int(t["max_depth"]), int(t["max_size"]), float(t["mean_size"]), float(t["mean_depth"])])
        out["games"].append({"black": game["black"], "moves": moves, "searches": searches, "outcome": game["outcome"]})
    return out


def main():
    root = sys.argv[1]
    n_games = int(sys.argv[2]) if len(sys.argv) > 2 else 6
    fixture = {}
    for key in SELECTED:
        paths = glob.glob(os.path.join(root, "experiments", "*[[]" + key + ";C4_6x7;*[]].zip"))
        assert len(paths) == 1, (key, paths)
        fixture[key] = extract(paths[0], n_games)
        for side in ("ai_a", "ai_b"):
            m = INSTANCE.match(fixture[key][side])
            fixture[key][side + "_config"] = None if m is None else {
                "search_time_limit": float(m.group(1)), "n_trees": int(m.group(3)), "n_playouts": int(m.group(4)),
                "variant": m.group(5), "device_memory": float(m.group(6)), "ucb_c": float(m.group(7)), "seed": int(m.group(8))}
    here = os.path.dirname(os.path.abspath(__file__))
    with open(os.path.join(here, "experiment_replays.json"), "w") as f:
        json.dump(fixture, f, separators=(",", ":"))
    print({k: sum(len(g["searches"]) for g in v["games"]) for k, v in fixture.items()})


if __name__ == "__main__":
    main()
