"""Launch tooling: expand an experiment's resource tree into tasks and run them.

* ``python -m steptronoss_b200.launch.mp_run exp.py [key=value ...]`` - every task of the experiment as a
  process group on this node (trainer, generation workers, router ...); when the critical tasks end, the
  rest is stopped.
* ``python -m steptronoss_b200.launch.build_scripts exp.py out_dir [key=value ...]`` - one shell script per
  task replica, for a cluster scheduler to run.
* ``python -m steptronoss_b200.launch.smartrun exp.py ...`` - ``torchrun`` whose node rank and master address
  come from a rendezvous in the experiment store (``NNODES`` nodes call it with the same ``EXP_ID``).

Reference: ``tools/mp_run.py``, ``tools/build_scripts.py``, ``tools/smartrun``.
"""
