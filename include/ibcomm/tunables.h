// Named integer knobs of single kernels (loads in flight, CTA counts, the
// split of the hybrid two-shot, ...).  A knob is looked up by name: a value
// set at run time (`SetTunable`, C API `ibcomm_set_tunable`) wins, then the
// environment variable of the same name, then the built-in default.  Unlike
// the reference's four IBCOMM_* variables these are not part of the contract;
// they exist so that a tuning run can sweep many settings inside one process
// (bench.py --tune) instead of one process launch per setting.
#pragma once

#include <string>

namespace ibcomm {

// Value of knob `name`; `dflt` when neither a run-time value nor an
// environment variable of that name exists.
int Tunable(const char* name, int dflt);
// Run-time override; `value` < 0 removes the override.
void SetTunable(const std::string& name, int value);
// Drops every run-time override.
void ClearTunables();

}  // namespace ibcomm
