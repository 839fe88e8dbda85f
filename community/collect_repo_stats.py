"""Contribution statistics for the project, as JSON or a markdown table.

The reference ships a GitHub-API collector for its community page (``community/collect_github_data.py``:
contributors, commits, issues and pull requests per period).  This tool reads the same figures that a checkout
can give without a network from ``git log``; with ``--github owner/repo`` (and a token in ``GITHUB_TOKEN``) it adds
the issue and pull-request counts from the REST API.

    python community/collect_repo_stats.py --since 2026-01-01 --format md
"""
from __future__ import annotations

import argparse
import collections
import datetime as dt
import json
import os
import subprocess
import sys


def git_log(repo: str, since: str | None) -> list[dict]:
    """One record per commit: hash, author, ISO date, files changed, lines added / removed."""
    cmd = ["git", "-C", repo, "log", "--numstat", "--date=short", "--pretty=format:@@%H|%an|%ad|%s"]
    if since:
        cmd.append(f"--since={since}")
    out = subprocess.run(cmd, check=True, capture_output=True, text=True).stdout
    commits, cur = [], None
    for line in out.splitlines():
        if line.startswith("@@"):
            h, author, date, subject = line[2:].split("|", 3)
            cur = {"hash": h, "author": author, "date": date, "subject": subject, "files": 0, "added": 0,
                   "removed": 0}
            commits.append(cur)
        elif line.strip() and cur is not None:
            parts = line.split("\t")
            if len(parts) == 3:
                cur["files"] += 1
                cur["added"] += int(parts[0]) if parts[0].isdigit() else 0  # "-" marks a binary file
                cur["removed"] += int(parts[1]) if parts[1].isdigit() else 0
    return commits


def summarise(commits: list[dict]) -> dict:
    per_author: dict = collections.defaultdict(lambda: {"commits": 0, "added": 0, "removed": 0})
    per_week: dict = collections.Counter()
    per_area: dict = collections.Counter()
    for c in commits:
        a = per_author[c["author"]]
        a["commits"] += 1
        a["added"] += c["added"]
        a["removed"] += c["removed"]
        y, w, _ = dt.date.fromisoformat(c["date"]).isocalendar()
        per_week[f"{y}-W{w:02d}"] += 1
        per_area[c["subject"].split(":", 1)[0][:24] if ":" in c["subject"][:28] else "(other)"] += 1
    return {
        "commits": len(commits),
        "contributors": len(per_author),
        "lines_added": sum(c["added"] for c in commits),
        "lines_removed": sum(c["removed"] for c in commits),
        "first": min((c["date"] for c in commits), default=None),
        "last": max((c["date"] for c in commits), default=None),
        "per_author": dict(sorted(per_author.items(), key=lambda kv: -kv[1]["commits"])),
        "per_week": dict(sorted(per_week.items())),
        "per_subject_prefix": dict(per_area.most_common(12)),
    }


def github_counts(slug: str, since: str | None) -> dict:
    """Open / closed issue and pull-request counts through the search API (needs network; token optional)."""
    import requests

    headers = {"Accept": "application/vnd.github+json"}
    if os.environ.get("GITHUB_TOKEN"):
        headers["Authorization"] = f"Bearer {os.environ['GITHUB_TOKEN']}"
    res = {}
    for kind in ("issue", "pr"):
        for state in ("open", "closed"):
            q = f"repo:{slug} is:{kind} is:{state}" + (f" created:>={since}" if since else "")
            r = requests.get("https://api.github.com/search/issues", params={"q": q, "per_page": 1}, headers=headers,
                             timeout=20)
            r.raise_for_status()
            res[f"{kind}_{state}"] = r.json().get("total_count", 0)
    return res


def to_markdown(s: dict) -> str:
    lines = [f"**{s['commits']} commits** by {s['contributors']} contributors, {s['first']} … {s['last']}; "
             f"+{s['lines_added']} / −{s['lines_removed']} lines", "", "| contributor | commits | added | removed |",
             "|---|---|---|---|"]
    for name, a in s["per_author"].items():
        lines.append(f"| {name} | {a['commits']} | {a['added']} | {a['removed']} |")
    lines += ["", "| week | commits |", "|---|---|"] + [f"| {w} | {n} |" for w, n in s["per_week"].items()]
    if "github" in s:
        lines += ["", "| GitHub | count |", "|---|---|"] + [f"| {k} | {v} |" for k, v in s["github"].items()]
    return "\n".join(lines)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--repo", default=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    ap.add_argument("--since", default=None, help="ISO date; default: the whole history")
    ap.add_argument("--github", default=None, metavar="OWNER/REPO", help="also query issue / PR counts (network)")
    ap.add_argument("--format", choices=("json", "md"), default="json")
    a = ap.parse_args(argv)
    s = summarise(git_log(a.repo, a.since))
    if a.github:
        try:
            s["github"] = github_counts(a.github, a.since)
        except Exception as e:  # noqa: BLE001 - offline machines still get the git figures
            s["github_error"] = str(e)
    print(to_markdown(s) if a.format == "md" else json.dumps(s, indent=2))
    return 0


if __name__ == "__main__":
    sys.exit(main())
