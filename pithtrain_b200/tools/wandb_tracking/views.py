"""Saved workspace views of a Weights & Biases project: which runs a shared link shows.

    python -m pithtrain_b200.tools.wandb_tracking.views list   <entity/project>
    python -m pithtrain_b200.tools.wandb_tracking.views show   <entity/project> <slug>
    python -m pithtrain_b200.tools.wandb_tracking.views create <entity/project> --name TITLE --runs RUN[,RUN...] [--like SLUG]
    python -m pithtrain_b200.tools.wandb_tracking.views edit   <entity/project> <slug> --runs RUN[,RUN...] [--name TITLE]
    python -m pithtrain_b200.tools.wandb_tracking.views delete <entity/project> <slug>

A project URL ending in ``?nw=<slug>`` opens the view stored under the name ``nw-<slug>-v``. Its spec is a JSON
document whose first run set has no filters (every run of the project is in the table) and a ``selections`` object
``{"root": 1, "tree": [...]}`` listing the run ids that are *hidden*; the visible runs are all the others. ``create``
copies panels and layout from an existing view (``--like``, else the project's first view, else a bare spec) and
rewrites only the hidden list; ``edit`` does the same in place, so the link stays valid. Same job as the reference's
helper (.agents/skills/wandb-tracking/scripts/views.py). The wandb client is imported lazily; ``main(argv, api=...,
graphql=...)`` accepts stand-ins, which is how the tests drive it.
"""

from __future__ import annotations

import argparse
import json
import secrets
import string
import sys
from dataclasses import dataclass
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

VIEW_KIND = "project-view"

LIST_QUERY = """
query ProjectViews($entityName: String!, $projectName: String!) {
  project(name: $projectName, entityName: $entityName) {
    allViews(viewType: "project-view") { edges { node { id name displayName spec } } }
  }
}
"""
UPSERT_MUTATION = """
mutation SaveView($input: UpsertViewInput!) { upsertView(input: $input) { view { id name displayName } inserted } }
"""
DELETE_MUTATION = """
mutation DropView($input: DeleteViewInput!) { deleteView(input: $input) { success } }
"""

GraphQL = Callable[[str, Dict[str, Any]], Dict[str, Any]]


def slug_of(view_name: str) -> Optional[str]:
    """``nw-<slug>-v`` -> ``<slug>``; ``None`` for views that are not workspace links."""
    if view_name.startswith("nw-") and view_name.endswith("-v") and len(view_name) > 5:
        return view_name[3:-2]
    return None


def name_of(slug: str) -> str:
    return f"nw-{slug}-v"


def _token(n: int) -> str:
    alphabet = string.ascii_lowercase + string.digits
    return "".join(secrets.choice(alphabet) for _ in range(n))


def bare_spec(run_set_id: str) -> Dict[str, Any]:
    """Smallest spec the workspace accepts: one unfiltered run set, automatic panels."""
    run_set = {
        "id": run_set_id, "name": "Run set", "enabled": True, "search": {"query": ""}, "grouping": [],
        "filters": {"filterFormat": "filterV2", "filters": []},
        "sort": {"keys": [{"key": {"section": "run", "name": "createdAt"}, "ascending": False}]},
        "runFeed": {"version": 2, "pageSize": 20, "onlyShowSelected": False, "columnVisible": {"run:name": False},
                    "columnPinned": {}, "columnWidths": {}, "columnOrder": [], "metricValences": {}},
        "selections": {"root": 1, "bounds": [], "tree": []}, "pinnedRunIds": [], "expandedRowAddresses": [],
    }
    return {"section": {
        "name": "", "version": 1, "openRunSet": 0, "openViz": True, "runSets": [run_set],
        "panelBankConfig": {"state": 1, "sections": [], "settings": {"showEmptySections": False, "sortAlphabetically": False}},
        "panelBankSectionConfig": {"__id__": "rps", "name": "Report Panels", "isOpen": False, "sorted": 0, "pinned": False,
                                   "panels": []},
        "customRunColors": {}, "customRunNames": {}, "workspaceSettings": {"linePlot": {}},
    }}


def hidden_ids(spec: Dict[str, Any]) -> List[str]:
    sel = spec["section"]["runSets"][0]["selections"]
    if sel.get("root") != 1:
        raise ValueError("this view selects runs explicitly (selections.root != 1); only hide-lists are handled")
    return list(sel.get("tree", []))


def split_runs(spec: Dict[str, Any], names_by_id: Dict[str, str]) -> Tuple[List[str], List[str]]:
    """``(visible, hidden)`` display names of a view, given every run of the project."""
    hidden = set(hidden_ids(spec))
    label = lambda i: names_by_id.get(i, i)  # noqa: E731
    return sorted(label(i) for i in names_by_id if i not in hidden), sorted(label(i) for i in hidden)


def with_visible(spec: Dict[str, Any], visible: Iterable[str], all_ids: Iterable[str]) -> Dict[str, Any]:
    """Copy of ``spec`` that shows exactly ``visible`` (run ids) out of ``all_ids``."""
    out = json.loads(json.dumps(spec))
    keep = set(visible)
    out["section"]["runSets"][0]["selections"] = {"root": 1, "bounds": [], "tree": sorted(set(all_ids) - keep)}
    return out


@dataclass
class View:
    id: str
    name: str
    title: str
    spec: Dict[str, Any]

    @property
    def slug(self) -> Optional[str]:
        return slug_of(self.name)


class ViewStore:
    """The saved views of one project, through a GraphQL executor ``graphql(document, variables) -> dict``."""

    def __init__(self, graphql: GraphQL, entity: str, project: str) -> None:
        self.graphql, self.entity, self.project = graphql, entity, project

    def all(self) -> List[View]:
        res = self.graphql(LIST_QUERY, {"entityName": self.entity, "projectName": self.project})
        out = []
        for edge in res["project"]["allViews"]["edges"]:
            n = edge["node"]
            try:
                spec = json.loads(n["spec"]) if isinstance(n["spec"], str) else dict(n["spec"])
            except (TypeError, json.JSONDecodeError):
                spec = {}
            out.append(View(n["id"], n["name"], n.get("displayName") or "", spec))
        return out

    def get(self, slug: str) -> View:
        for v in self.all():
            if v.name == name_of(slug):
                return v
        raise SystemExit(f"no view with link ?nw={slug} in {self.entity}/{self.project}")

    def save(self, spec: Dict[str, Any], title: str, existing: Optional[View] = None) -> Tuple[str, bool]:
        """Insert a new view or overwrite ``existing``; returns ``(slug, inserted)``."""
        fields: Dict[str, Any] = {"entityName": self.entity, "projectName": self.project, "type": VIEW_KIND,
                                  "displayName": title, "spec": json.dumps(spec)}
        if existing is not None:
            fields.update(id=existing.id, name=existing.name)
            slug = existing.slug or existing.name
        else:
            slug = _token(11)
            fields.update(name=name_of(slug), createdUsing="WANDB_SDK")
        res = self.graphql(UPSERT_MUTATION, {"input": fields})
        return slug, bool(res["upsertView"]["inserted"])

    def delete(self, view: View) -> bool:
        return bool(self.graphql(DELETE_MUTATION, {"input": {"id": view.id}})["deleteView"]["success"])


def _run_ids(selectors: Sequence[str], names_by_id: Dict[str, str]) -> List[str]:
    ids = []
    for s in selectors:
        if s in names_by_id:
            ids.append(s)
            continue
        hits = [i for i, n in names_by_id.items() if n == s]
        if len(hits) != 1:
            raise SystemExit(f"{len(hits)} runs are called {s!r}: use run ids" if hits else f"no run {s!r} in the project")
        ids.append(hits[0])
    return ids


def _describe(view: View, names_by_id: Dict[str, str]) -> List[str]:
    lines = [f"{view.title!r}  ?nw={view.slug or '-'}  ({view.name})"]
    try:
        visible, hidden = split_runs(view.spec, names_by_id)
        lines += [f"  visible: {', '.join(visible) or '-'}", f"  hidden : {', '.join(hidden) or '-'}"]
    except (KeyError, IndexError, ValueError) as e:
        lines.append(f"  (no hide-list in this view: {e})")
    return lines


def main(argv: Optional[Sequence[str]] = None, api=None, graphql: Optional[GraphQL] = None) -> int:
    ap = argparse.ArgumentParser(prog="views", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    sub.add_parser("list").add_argument("project")
    for c in ("show", "delete"):
        p = sub.add_parser(c)
        p.add_argument("project"); p.add_argument("slug")
    p = sub.add_parser("create")
    p.add_argument("project"); p.add_argument("--name", required=True); p.add_argument("--runs", required=True)
    p.add_argument("--like", help="slug of the view whose panels and layout are copied")
    p = sub.add_parser("edit")
    p.add_argument("project"); p.add_argument("slug"); p.add_argument("--runs", required=True); p.add_argument("--name")
    a = ap.parse_args(argv)

    if api is None:
        from .runs import _api

        api = _api()
    if graphql is None:
        graphql = api._service_api.execute_graphql  # the client's own executor
    entity, project = a.project.split("/", 1)
    store = ViewStore(graphql, entity, project)
    names_by_id = {r.id: r.name for r in api.runs(a.project)}

    if a.cmd == "list":
        for v in store.all():
            print("\n".join(_describe(v, names_by_id)))
        return 0
    if a.cmd == "show":
        print("\n".join(_describe(store.get(a.slug), names_by_id)))
        return 0
    if a.cmd == "delete":
        v = store.get(a.slug)
        ok = store.delete(v)
        print(f"deleted {v.title!r} (?nw={a.slug}): {'ok' if ok else 'refused'}")
        return 0 if ok else 1

    visible = _run_ids(a.runs.split(","), names_by_id)
    if a.cmd == "edit":
        target = store.get(a.slug)
        spec = with_visible(target.spec, visible, names_by_id)
        slug, inserted = store.save(spec, a.name or target.title, existing=target)
    else:
        views = store.all()
        base = store.get(a.like) if a.like else next((v for v in views if v.spec.get("section", {}).get("runSets")), None)
        spec = with_visible(base.spec if base else bare_spec(_token(9)), visible, names_by_id)
        spec["section"]["runSets"][0]["id"] = _token(9)
        slug, inserted = store.save(spec, a.name)
    print(f"{'created' if inserted else 'updated'} ?nw={slug}: https://wandb.ai/{a.project}?nw={slug}")
    print("  visible: " + ", ".join(sorted(names_by_id[i] for i in visible)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
