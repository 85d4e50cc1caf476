"""Link-matrix topology with optional shared-bandwidth switch groups.

``links[dst][src]`` is the integer bandwidth (chunks per round) of the
directed link ``src -> dst``.  A switch is a tuple ``(srcs, dsts, bw, name)``
limiting the sum of traffic from any of ``srcs`` to any of ``dsts``.

Parity: reference ``msccl/topologies/topology.py:4-41``.
"""


class Topology:
    def __init__(self, name, links, switches=None):
        self.name = name
        self.links = links
        self.switches = list(switches) if switches else []
        for _srcs, _dsts, bw, sw_name in self.switches:
            if bw == 0:
                raise ValueError(f'Switch {sw_name} has zero bandwidth, but switch bandwidths must be '
                                 'strictly positive. Please encode connectedness in links.')
            if bw < 0:
                raise ValueError(f'Switch {sw_name} has a negative bandwidth of {bw}. '
                                 'Bandwidth must be strictly positive.')

    def num_nodes(self):
        return len(self.links)

    def nodes(self):
        return range(len(self.links))

    def link(self, src, dst):
        return self.links[dst][src]

    def sources(self, dst):
        return (src for src, bw in enumerate(self.links[dst]) if bw > 0)

    def destinations(self, src):
        return (dst for dst, row in enumerate(self.links) if row[src] > 0)

    def bandwidth_constraints(self):
        """Yield ``(srcs, dsts, bw, name)``: first one per link, then the switches."""
        for dst, row in enumerate(self.links):
            for src, bw in enumerate(row):
                if bw > 0:
                    yield [src], [dst], bw, f'{src}→{dst}'
        yield from self.switches

    def __repr__(self):
        return f'Topology({self.name!r}, nodes={self.num_nodes()}, switches={len(self.switches)})'
