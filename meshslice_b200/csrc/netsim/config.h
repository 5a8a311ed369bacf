// netsim: system description files.
//
// The reference describes its simulated machine in SST Python scripts and ini files
// (tests/runVanadis.py, rdmaNic.py, memory.py, hbmmemory.py, hbmdevice.ini, hbmsystem.ini),
// steered by environment variables.  Here one ini file holds the sections [run], [network],
// [nic], [memory], [host] and [mpi]; command-line options override it.  Unknown sections or keys
// are errors, so a typo cannot silently fall back to a default.
#pragma once
#include <string>

#include "scenarios.h"

namespace netsim {

// Applies `path` to `cfg`.  Returns false and sets `error` ("file:line: message") on failure.
bool load_config(const std::string& path, ScenarioConfig& cfg, std::string& error);
// Applies one "section.key=value" assignment (also used for --set on the command line).
bool apply_setting(const std::string& section, const std::string& key, const std::string& value, ScenarioConfig& cfg,
                   std::string& error);
// The effective configuration as ini text (what a run used).
std::string dump_config(const ScenarioConfig& cfg);

}  // namespace netsim
