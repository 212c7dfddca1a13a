"""Stage the reference's own CPU implementation of the path under oracle/_ref/ (git-ignored).  TEST INFRASTRUCTURE ONLY.

    python oracle/build_ref.py [--reference <checkout of the reference>]      (or the SPGT_REFERENCE environment variable)

The reference's CPU path is two pure-PyTorch files, network/layer.py and network/model.py ("GT" model family); they
import nothing but torch and each other (as package ``SpGT``).  Python has no compile step, so "building" the
reference here means copying those two files, unmodified, from the checkout into oracle/_ref/SpGT/network/ next to
empty package markers.  The copy is never committed (oracle/_ref/ is ignored by git); it exists so that the
benchmark's CPU legs can time the reference's own code on machines that have no checkout of the reference.  When no
checkout is available the benchmark falls back to the restatement in oracle/gt_oracle.py and says so.
"""
from __future__ import annotations

import argparse
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, '_ref')
FILES = (('network', 'layer.py'), ('network', 'model.py'))


def default_reference() -> str:
    """SPGT_REFERENCE, else a directory named `reference` beside the repository."""
    return os.environ.get('SPGT_REFERENCE') or os.path.join(os.path.dirname(os.path.dirname(HERE)), 'reference')


def build(reference: str | None = None, verbose: bool = False) -> bool:
    """Returns True when oracle/_ref holds the reference's files afterwards (copied now or earlier)."""
    reference = reference or default_reference()
    have = all(os.path.isfile(os.path.join(DEST, 'SpGT', *f)) for f in FILES)
    if not all(os.path.isfile(os.path.join(reference, *f)) for f in FILES):
        if verbose:
            print(f'no reference checkout at {reference}: oracle/_ref {"kept as is" if have else "not built"}')
        return have
    for sub in ('SpGT', os.path.join('SpGT', 'network')):
        os.makedirs(os.path.join(DEST, sub), exist_ok=True)
        with open(os.path.join(DEST, sub, '__init__.py'), 'w'):
            pass
    for f in FILES:
        shutil.copyfile(os.path.join(reference, *f), os.path.join(DEST, 'SpGT', *f))
    if verbose:
        print(f'copied {len(FILES)} files from {reference} to {DEST}')
    return True


if __name__ == '__main__':
    ap = argparse.ArgumentParser()
    ap.add_argument('--reference', default=None)
    ok = build(ap.parse_args().reference, verbose=True)
    sys.exit(0 if ok else 1)
