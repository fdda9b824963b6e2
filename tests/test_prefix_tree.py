"""Behaviour of the prefix cache index as restated in retrograd_b200/prefix_tree.py, on the scenarios the
reference checks its own tree with (crates/retrograd-infer/src/kv.rs:549-690): edge walks and splits,
exact and mid-sequence hits, pins and LRU eviction, pruning, namespaces."""
from oracle.prefix_tree import PrefixTree


def _tree(*paths):
    tree = PrefixTree()
    for i, path in enumerate(paths):
        tree.insert(0, path, i + 1)
    return tree


def _hit(found):
    return None if found is None else (found[0].slot, found[1])


def test_lookup_walks_whole_edges_and_offers_mid_sequence_hits_only_when_allowed():
    tree = _tree([1, 2, 3, 4], [1, 2, 9, 9])
    assert _hit(tree.longest_prefix(0, [1, 2, 3, 4, 5], True)) == (1, 4)              # the first path's own boundary
    # leaves the second path inside its edge: three shared tokens from its slot, or the fork (depth 2) when only boundaries count
    assert _hit(tree.longest_prefix(0, [1, 2, 9, 8], True)) == (2, 3)
    assert tree.longest_prefix(0, [1, 2, 9, 8], False)[1] == 2
    tree = _tree([1, 2, 3, 4])
    assert _hit(tree.longest_prefix(0, [1, 2], True)) == (1, 2)                         # the prompt ends inside an edge
    assert tree.longest_prefix(0, [1, 2], False) is None
    # no child continues the prompt at a fork without a slot: the shared prefix is still served from a child's slot
    tree = _tree([1, 2, 3], [1, 2, 9])
    has_slot = lambda node, hit: node.slot is not None
    assert tree.longest_prefix(0, [1, 2, 7], True, has_slot)[1] == 2
    assert tree.longest_prefix(0, [1, 2, 7], False, has_slot) is None
    # a node the backend cannot use is passed over for the shallower one
    tree = _tree([1, 2, 3], [1, 2, 3, 4])
    assert _hit(tree.longest_prefix(0, [1, 2, 3, 4, 5], False, lambda node, hit: node.slot != 2)) == (1, 3)


def test_a_path_attaches_one_slot_and_a_pin_keeps_it_from_eviction():
    tree = _tree([7, 7, 7])
    node, attached = tree.insert(0, [7, 7, 7], 42)
    assert not attached and node.slot == 1            # the caller releases slot 42 itself
    pin = tree.pin_at(0, [7, 7, 7])
    assert pin is not None and tree.eviction_candidate() is None
    assert tree.unpin(pin) and tree.eviction_candidate() is node
    assert not tree.unpin(pin)                         # ids are never reused
    assert tree.pin_at(0, [8, 8]) is None


def test_eviction_takes_the_least_recently_used_slot():
    tree = _tree([1, 1], [2, 2], [3, 3])
    first = tree.find_exact(0, [1, 1])
    tree.touch(first)                                  # now the most recent
    assert tree.eviction_candidate().slot == 2
    victim = tree.eviction_candidate()
    tree.attach_snapshot(victim, b"x" * 64)
    tree.detach_slot(victim)                           # swapped out: host bytes, no pool cells
    assert tree.eviction_candidate().slot == 3
    assert tree.snapshot_eviction_candidate() is victim and tree.snapshot_bytes == 64


def test_clear_returns_every_slot_and_forgets_the_snapshots():
    tree = _tree([1], [1, 2])
    tree.attach_snapshot(tree.find_exact(0, [1, 2]), bytes(100))
    assert tree.snapshot_bytes == 100
    assert sorted(tree.clear()) == [1, 2]
    assert tree.node_count() == 0 and tree.snapshot_bytes == 0


def test_remove_prunes_the_emptied_branch_up_to_the_root():
    tree = _tree([1, 2], [5, 6])
    node, _ = tree.insert(0, [1, 2], 9)
    tree.remove(node)
    assert tree.node_count() == 1
    assert tree.longest_prefix(0, [1, 2, 3], True) is None
    _, attached = tree.insert(0, [7, 8], 3)
    assert attached and tree.node_count() == 2
    # a fork node survives while another branch hangs from it
    tree = _tree([1, 2, 3], [1, 2, 9])
    tree.remove(tree.find_exact(0, [1, 2, 3]))
    assert tree.node_count() == 2 and _hit(tree.longest_prefix(0, [1, 2, 9], False)) == (2, 3)


def test_namespaces_share_nothing_and_drop_alone():
    tree = PrefixTree()
    tree.insert(0, [1, 2, 3, 4], 1)
    tree.insert(7, [1, 2, 3, 4], 2)
    tree.insert(7, [1, 2, 9], 3)
    assert _hit(tree.longest_prefix(0, [1, 2, 3, 4, 5], False)) == (1, 4)
    assert _hit(tree.longest_prefix(7, [1, 2, 3, 4, 5], False)) == (2, 4)
    assert tree.longest_prefix(8, [1, 2, 3, 4], True) is None
    assert tree.node_count() == 4
    pin = tree.pin_at(7, [1, 2, 9])
    assert sorted(tree.drop_namespace(7)) == [2, 3]
    assert not tree.unpin(pin)
    assert tree.longest_prefix(7, [1, 2, 3, 4], True) is None
    assert tree.node_count() == 1 and tree.resident_slots() == [1] and tree.resident_cells() == 4
    tree.insert(7, [5, 6], 4)
    assert tree.node_count() == 2
