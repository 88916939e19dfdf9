"""Write the reference's two shipped layout configurations as JSON fixtures.

    SUBSTATION_REF=/path/to/substation python tests/golden/make_layout_fixtures.py

Reads pytorch_module/layouts-bert-b8-l512-h16-e1024.pickle and
pytorch_module/layouts-bert-b96-l128-h16-e1024.pickle (plain dicts of strings,
schema of config_selection/optimize.py:443-493) and dumps them unchanged to
tests/golden/layouts_*.json so that tests on a machine without the reference
tree can load them.
"""

import json
import os
import sys
import pickle

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get('SUBSTATION_REF') or sys.exit('set SUBSTATION_REF to a checkout of spcl/substation')

for tag in ('b8-l512', 'b96-l128'):
    with open(os.path.join(REF, 'pytorch_module', f'layouts-bert-{tag}-h16-e1024.pickle'), 'rb') as f:
        d = pickle.load(f)
    out = os.path.join(HERE, f'layouts_{tag.replace("-", "_")}.json')
    with open(out, 'w') as f:
        json.dump(d, f, indent=1, sort_keys=True)
    print(out)
