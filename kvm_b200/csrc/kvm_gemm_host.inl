// Host planning of the tensor-core tasks (placeholder).
static int kvm_plan_tc(KvmExec* h, int first_task) { (void)h; (void)first_task; return 0; }
