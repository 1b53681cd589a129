#!/bin/bash
# Runs the six Open-LLM-leaderboard tasks of EleutherAI's lm-evaluation-harness on a model exported with
# `python -m llmc_b200.utils.export_hf` and prints the summary (reference: dev/eval/run_eval.sh).
#
#   ./llm.c_b200/eval/run_eval.sh <hf model name or exported directory> <result name>
#
# Needs a checkout of lm-evaluation-harness (commit b281b0921b636bc36ad05c0b0b0763bd6dd43463, `pip install -e .`) next to the
# repository root, and network access for the task data; neither is part of this repository.
set -e
if [ -z "$1" ] || [ -z "$2" ]; then
    echo "usage: $0 <hf model name or path to an exported model> <result name>"
    exit 1
fi
if [ ! -d lm-evaluation-harness ]; then
    echo "lm-evaluation-harness/ not found in $(pwd): clone it here first (see the header of this script)"
    exit 1
fi
MODEL="$(realpath -s "$1")"
RESULT="$2"
echo "Evaluating model $MODEL"
echo "Saving results to ./lm-evaluation-harness/results/$RESULT"
ARGS="--model hf-causal-experimental --model_args pretrained=$MODEL,use_accelerate=True,trust_remote_code=True --batch_size 1 --no_cache --write_out --device cuda"
MMLU=$(python - <<'PY'
subjects = """abstract_algebra anatomy astronomy business_ethics clinical_knowledge college_biology college_chemistry college_computer_science
college_mathematics college_medicine college_physics computer_security conceptual_physics econometrics electrical_engineering
elementary_mathematics formal_logic global_facts high_school_biology high_school_chemistry high_school_computer_science
high_school_european_history high_school_geography high_school_government_and_politics high_school_macroeconomics high_school_mathematics
high_school_microeconomics high_school_physics high_school_psychology high_school_statistics high_school_us_history
high_school_world_history human_aging human_sexuality international_law jurisprudence logical_fallacies machine_learning management
marketing medical_genetics miscellaneous moral_disputes moral_scenarios nutrition philosophy prehistory professional_accounting
professional_law professional_medicine professional_psychology public_relations security_studies sociology us_foreign_policy virology
world_religions""".split()
print(",".join("hendrycksTest-" + s for s in subjects))
PY
)
cd lm-evaluation-harness
python main.py $ARGS --tasks truthfulqa_mc --output_path results/$RESULT/truthfulqa_0shot.json
python main.py $ARGS --tasks winogrande --num_fewshot 5 --output_path results/$RESULT/winogrande_5shot.json
python main.py $ARGS --tasks arc_challenge --num_fewshot 25 --output_path results/$RESULT/arc_challenge_25shot.json
python main.py $ARGS --tasks hellaswag --num_fewshot 10 --output_path results/$RESULT/hellaswag_10shot.json
python main.py $ARGS --tasks gsm8k --num_fewshot 5 --output_path results/$RESULT/gsm8k_5shot.json
python main.py $ARGS --tasks $MMLU --num_fewshot 5 --output_path results/$RESULT/mmlu_5shot.json
cd ..
python -m llmc_b200.eval.summarize_eval lm-evaluation-harness/results/$RESULT
