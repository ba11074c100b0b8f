# Front door for people used to `make`: every target delegates to the Python build driver (cai_b200/_build.py), which
# compiles the sm_100a kernel library, the GPU-free host library and the tools in-tree with nvcc / g++.
PYTHON ?= python

.PHONY: all host test gputest demo predict interpret clean

all:            ## kernels (sm_100a), host library, tools
	$(PYTHON) -m cai_b200._build

host:           ## GPU-free parts only: plan compiler, verifier, pricing backends, oracle, tools
	$(PYTHON) -c "from cai_b200 import _build; _build.build_host()"

test: host      ## C++ self-test (also under ASan / UBSan via pytest) and the CPU test suite
	./bin/cai_selftest
	$(PYTHON) -m pytest tests -q -m "not gpu"

gputest: all    ## kernels against fp32 PyTorch, engine against the fp32 model, multi-GPU layouts (needs B200s)
	$(PYTHON) -m pytest tests -q -m gpu

# End to end without a GPU: lint and verify the 220,032-rank configuration, compile sample ranks, replay stage 0 with
# the reference's cost model, train the fp64 oracle; then the B200 part: an executable plan of the benchmark model,
# verified (hazards, cross-rank buffer reuse) and priced with measured kernel costs.
demo: host
	@echo "== lint full220k =="
	./bin/topology_linter configs/full220k.cfg
	@echo "== verify all 220,032 ranks pre-launch =="
	./bin/plan_verify configs/full220k.cfg
	@echo "== compile 220,032-GPU sample =="
	./bin/plan_compiler configs/full220k.cfg out/full
	@echo "== replay stage 0 of the 220k plan (analytic backend) =="
	./bin/trainer out/full/plan.rank000000.bin out/full/topology.bin --steps 5
	@echo "== all three stages of small.cfg replayed together (no bubble formula) =="
	./bin/plan_compiler configs/small.cfg out/small --all --quiet > /dev/null
	./bin/trainer out/small/plan.rank000000.bin out/small/topology.bin --pipeline
	@echo "== train the fp64 oracle on CPU =="
	./bin/reftrain --steps 400
	@echo "== executable plan for 8 B200s: compile, verify, predict =="
	./bin/plan_compiler configs/b200_tp8.cfg out/tp8 --exec --all
	./bin/plan_verify configs/b200_tp8.cfg --dir out/tp8 --exec
	./bin/trainer out/tp8/plan.rank000000.bin out/tp8/topology.bin --steps 1 --backend calibrated

predict: host   ## rank the executable layouts of CONFIG on GPUS B200s by predicted step time
	$(PYTHON) -m cai_b200.plan.advise $(or $(CONFIG),configs/b200_tp8.cfg) --gpus $(or $(GPUS),8)

interpret: host ## run CONFIG's executable plans on the host, every rank in one process, next to the fp32 model (small models)
	$(PYTHON) -m cai_b200.models.plan_interpreter $(or $(CONFIG),configs/tiny_mp.cfg) $(if $(ORDER),--order $(ORDER))

clean:
	rm -rf build bin out cai_b200/lib
