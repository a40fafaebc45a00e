"""Generate ``connector_config.json`` from the reference's own connector helpers
(python/pegaflow/connector/common.py: PegaConnectorMode, TpShardTopology, resolve_instance_id,
derive_namespace, detect_mla, reconcile_hybrid_hit), imported with the reference's ``unit_stubs``
in place of its native extension.  Inputs are written next to the outputs so that the test can
rebuild the same fake vLLM configs without the reference.

    PEGAFLOW_REFERENCE=<checkout> python tests/golden/gen_connector_config.py
"""
import json
import os
import random
import sys

_REPO = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
REF = os.environ.get("PEGAFLOW_REFERENCE", os.path.join(os.path.dirname(_REPO), "reference"))
sys.path.insert(0, os.path.join(REF, "python"))
from tests.unit_stubs import install_connector_unit_stubs  # noqa: E402  (the reference's tests package)

install_connector_unit_stubs()
from pegaflow.connector import common as ref  # noqa: E402

import importlib.util  # noqa: E402

_spec = importlib.util.spec_from_file_location("connector_config_cases",
                                               os.path.join(_REPO, "tests", "connector_config_cases.py"))
cases = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(cases)


def main():
    out = cases.run_all(ref, random.Random(20260101))
    out["cache_groups"] = cases.run_cache_groups(ref)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "connector_config.json")
    with open(path, "w") as f:
        json.dump(out, f, sort_keys=True)
        f.write("\n")
    print(path, {k: len(v) for k, v in out.items()})


if __name__ == "__main__":
    main()
