"""Host-side mirror of the reference's prefix cache index (`PrefixTree`, crates/retrograd-infer/src/kv.rs:140-537):
a compressed trie over the token sequences of finished requests, one trie per namespace (the adapter a
path was decoded under), whose nodes remember which dormant engine slot holds the KV of `[0, depth)`.
The tree stays with the caller; what reaches the engine are its decisions - "copy `[0, hit)` from slot s
to the new request's slot" (`retro_engine_seq_cp`) and "release slot s" (`retro_engine_seq_rm`). This
restatement lets Python-driven workloads make those decisions the way the Rust scheduler does.

Behaviour restated (line numbers in kv.rs):
  * `longest_prefix` walks whole edges; the deepest usable node on the way is an exact hit (`hit == depth`,
    a whole-slot copy). Where the walk stops - the prompt diverges, ends inside an edge, or the branch has no
    slot - a mid-sequence hit of `pos + matched` tokens may be served from the deepest slot-bearing node of
    the continuing subtree, if `partial_ok` and it is longer than the exact hit (:213-266).
  * `insert` splits an edge where a new path diverges and attaches the slot at the end node unless that
    node already owns one (then the caller releases the slot it passed) (:291-339).
  * pins are counted per node, their ids never reused; eviction candidates are the least recently used
    unpinned nodes that own a slot (or, for host bytes, only a snapshot) (:371-435).
  * `remove` drops a node's payload and prunes it and every ancestor left without children, payload and
    pins (:437-460); namespaces share nothing and can be dropped alone (:492-524).

Test infrastructure, like the rest of this folder: the shipped library never imports it.
"""
from __future__ import annotations

from typing import Callable, Iterator, Optional, Sequence


class _Node:
    __slots__ = ("edge", "parent", "depth", "slot", "snapshot", "last_use", "pins", "children")

    def __init__(self, edge: list[int], parent: Optional["_Node"], depth: int) -> None:
        self.edge, self.parent, self.depth = edge, parent, depth
        self.slot: Optional[int] = None
        self.snapshot: Optional[bytes] = None
        self.last_use = 0
        self.pins = 0
        self.children: dict[int, _Node] = {}

    @property
    def is_root(self) -> bool:
        return self.parent is None


def _common(edge: Sequence[int], tokens: Sequence[int]) -> int:
    n = 0
    for a, b in zip(edge, tokens):
        if a != b:
            break
        n += 1
    return n


class PrefixTree:
    def __init__(self) -> None:
        self._roots: dict[int, _Node] = {}
        self._clock = 0
        self._next_pin = 1
        self._pins: dict[int, _Node] = {}
        self.snapshot_bytes = 0

    # ---- helpers
    def _tick(self) -> int:
        self._clock += 1
        return self._clock

    def _nodes(self, root: Optional[_Node] = None) -> Iterator[_Node]:
        stack = [root] if root is not None else list(self._roots.values())
        while stack:
            node = stack.pop()
            if not node.is_root:
                yield node
            stack.extend(node.children.values())

    # ---- lookup
    def longest_prefix(self, ns: int, tokens: Sequence[int], partial_ok: bool,
                       usable: Callable[[_Node, int], bool] = lambda node, hit: True) -> Optional[tuple[_Node, int]]:
        cur = self._roots.get(ns)
        if cur is None:
            return None
        best: Optional[tuple[_Node, int]] = None
        pos = 0
        while True:
            if cur.depth > 0 and usable(cur, cur.depth):
                best = (cur, cur.depth)
            child = cur.children.get(tokens[pos]) if pos < len(tokens) else None
            matched = _common(child.edge, tokens[pos:]) if child is not None else 0
            if child is not None and matched == len(child.edge):
                cur, pos = child, pos + matched
                continue
            if partial_ok:
                below = child if child is not None else next(iter(sorted(cur.children.items())), (None, None))[1]
                hit = pos + matched
                if below is not None and hit > 0 and (best is None or hit > best[1]):
                    holder = self._deepest_slot(below)
                    if holder is not None and usable(holder, hit):
                        best = (holder, hit)
            return best

    def _deepest_slot(self, node: _Node) -> Optional[_Node]:
        best = None
        stack = [node]
        while stack:
            cur = stack.pop()
            if cur.slot is not None and (best is None or cur.depth > best.depth):
                best = cur
            stack.extend(cur.children.values())
        return best

    def find_exact(self, ns: int, tokens: Sequence[int]) -> Optional[_Node]:
        cur = self._roots.get(ns)
        pos = 0
        while cur is not None and pos < len(tokens):
            child = cur.children.get(tokens[pos])
            if child is None or list(tokens[pos:pos + len(child.edge)]) != child.edge:
                return None
            cur, pos = child, pos + len(child.edge)
        return cur if cur is not None and not cur.is_root else None

    # ---- updates
    def touch(self, node: _Node) -> None:
        node.last_use = self._tick()

    def insert(self, ns: int, tokens: Sequence[int], slot: int) -> tuple[_Node, bool]:
        tokens = list(tokens)
        cur = self._roots.setdefault(ns, _Node([], None, 0))
        pos = 0
        while pos < len(tokens):
            first = tokens[pos]
            child = cur.children.get(first)
            if child is None:
                child = _Node(tokens[pos:], cur, len(tokens))
                cur.children[first] = child
                cur, pos = child, len(tokens)
                continue
            matched = _common(child.edge, tokens[pos:])
            if matched < len(child.edge):
                # the new path leaves this edge part-way: a node at the fork takes the shared head
                mid = _Node(child.edge[:matched], cur, cur.depth + matched)
                child.edge = child.edge[matched:]
                child.parent = mid
                mid.children[child.edge[0]] = child
                cur.children[first] = mid
                cur = mid
            else:
                cur = child
            pos += matched
        attached = not cur.is_root and cur.slot is None
        if attached:
            cur.slot = slot
            cur.last_use = self._tick()
        return cur, attached

    def attach_snapshot(self, node: _Node, snapshot: bytes) -> None:
        if node.snapshot is not None:
            self.snapshot_bytes -= len(node.snapshot)
        node.snapshot = snapshot
        self.snapshot_bytes += len(snapshot)

    def detach_slot(self, node: _Node) -> None:
        node.slot = None

    def pin_node(self, node: _Node) -> int:
        node.pins += 1
        node.last_use = self._tick()
        pin = self._next_pin
        self._next_pin += 1
        self._pins[pin] = node
        return pin

    def pin_at(self, ns: int, tokens: Sequence[int]) -> Optional[int]:
        node = self.find_exact(ns, tokens)
        return self.pin_node(node) if node is not None else None

    def unpin(self, pin: int) -> bool:
        node = self._pins.pop(pin, None)
        if node is None:
            return False
        node.pins -= 1
        return True

    def _lru(self, eligible: Callable[[_Node], bool]) -> Optional[_Node]:
        found = [n for n in self._nodes() if n.pins == 0 and eligible(n)]
        return min(found, key=lambda n: n.last_use) if found else None

    def eviction_candidate(self) -> Optional[_Node]:
        return self._lru(lambda n: n.slot is not None)

    def snapshot_eviction_candidate(self) -> Optional[_Node]:
        return self._lru(lambda n: n.slot is None and n.snapshot is not None)

    def remove(self, node: _Node) -> None:
        if node.snapshot is not None:
            self.snapshot_bytes -= len(node.snapshot)
            node.snapshot = None
        node.slot = None
        while not node.is_root and not node.children and node.slot is None and node.snapshot is None and node.pins == 0:
            parent = node.parent
            del parent.children[node.edge[0]]
            node.parent = None
            node = parent

    # ---- inventory
    def resident_slots(self) -> list[int]:
        return [n.slot for n in self._nodes() if n.slot is not None]

    def resident_cells(self) -> int:
        return sum(n.depth for n in self._nodes() if n.slot is not None)

    def node_count(self) -> int:
        return sum(1 for _ in self._nodes())

    def clear(self) -> list[int]:
        slots = self.resident_slots()
        self._roots.clear()
        self._pins.clear()
        self.snapshot_bytes = 0
        return slots

    def drop_namespace(self, ns: int) -> list[int]:
        root = self._roots.pop(ns, None)
        if root is None:
            return []
        gone = list(self._nodes(root))
        for node in gone:
            if node.snapshot is not None:
                self.snapshot_bytes -= len(node.snapshot)
        dropped = {id(n) for n in gone}
        self._pins = {pin: n for pin, n in self._pins.items() if id(n) not in dropped}
        return [n.slot for n in gone if n.slot is not None]
