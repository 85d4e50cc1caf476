"""On-disk cache of synthesis results, keyed by (topology, collective, instance).

A solver call can take minutes (the Pareto searches of the synthesis guide spend up to two minutes in
one instance), and the same instances come up again whenever plans are registered or a search is
repeated.  With ``MSCCL_SYNTH_CACHE=<directory>`` every solved instance is written there as an ordinary
``.msccl.json`` algorithm file (loadable by every tool that takes algorithm files), unsatisfiable ones as
a one-line marker, and later calls with an equal topology, collective and instance return the stored
answer.  The key is the SHA-256 of the JSON form of the three objects, so a renamed but otherwise equal
topology is a different key, as it is a different algorithm name.

The reference keeps results only when asked to (``-o`` / ``--save-eagerly`` of ``msccl solve``, reference
``msccl/cli/solve.py:63,83-84``); this cache is an addition.
"""
import hashlib
import json
import os

from msccl.serialization import MSCCLDecoder, MSCCLEncoder

_UNSAT = {'msccl_type': 'unsatisfiable'}


class SynthesisCache:
    def __init__(self, directory):
        self.directory = directory
        self.hits = 0
        self.misses = 0

    def key(self, topology, collective, instance):
        text = MSCCLEncoder().encode({'topology': topology, 'collective': collective, 'instance': instance})
        return hashlib.sha256(text.encode()).hexdigest()

    def _path(self, key):
        return os.path.join(self.directory, key + '.msccl.json')

    def lookup(self, topology, collective, instance):
        """``(True, algorithm or None)`` if the instance was solved before (None = unsatisfiable), else ``(False, None)``."""
        path = self._path(self.key(topology, collective, instance))
        try:
            with open(path) as f:
                text = f.read()
        except OSError:
            self.misses += 1
            return False, None
        try:
            if json.loads(text) == _UNSAT:
                self.hits += 1
                return True, None
            algo = MSCCLDecoder().decode(text)
        except (ValueError, KeyError, TypeError):
            self.misses += 1                       # damaged entry: solve again, the store below replaces it
            return False, None
        self.hits += 1
        return True, algo

    def store(self, topology, collective, instance, algorithm):
        os.makedirs(self.directory, exist_ok=True)
        path = self._path(self.key(topology, collective, instance))
        text = json.dumps(_UNSAT) if algorithm is None else MSCCLEncoder().encode(algorithm)
        tmp = f'{path}.{os.getpid()}.tmp'
        with open(tmp, 'w') as f:
            f.write(text)
        os.replace(tmp, path)                      # readers never see a half-written file


_caches = {}


def active_cache():
    """The cache named by ``MSCCL_SYNTH_CACHE``, or None when the variable is unset or empty."""
    directory = os.environ.get('MSCCL_SYNTH_CACHE')
    if not directory:
        return None
    if directory not in _caches:
        _caches[directory] = SynthesisCache(directory)
    return _caches[directory]
