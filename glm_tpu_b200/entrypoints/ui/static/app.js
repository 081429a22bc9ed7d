// Loopback chat workspace: polls /api/state, posts actions to /api/chat.  No external resources.
"use strict";
const $ = (id) => document.getElementById(id);
let state = { chats: [], jobs: [], error: null };
let current = null;

function hexId() {
  const bytes = new Uint8Array(16);
  crypto.getRandomValues(bytes);
  return Array.from(bytes, (b) => b.toString(16).padStart(2, "0")).join("");
}

async function post(body) {
  const res = await fetch("/api/chat", {
    method: "POST",
    headers: { "Content-Type": "application/json", "X-GLM-UI": "1" },
    body: JSON.stringify(body),
  });
  const data = await res.json();
  if (!res.ok) throw new Error(data.error || "request failed");
  return data;
}

function el(tag, cls, text) {
  const node = document.createElement(tag);
  if (cls) node.className = cls;
  if (text !== undefined) node.textContent = text;
  return node;
}

function render() {
  const list = $("chat-list");
  list.replaceChildren();
  for (const chat of state.chats) {
    const item = el("li", chat.id === current ? "active" : "", chat.title);
    item.addEventListener("click", () => { current = chat.id; render(); });
    list.appendChild(item);
  }
  const banner = $("banner");
  banner.hidden = !state.error;
  banner.textContent = state.error || "";
  $("session-info").textContent = state.model ? `${state.model} · ${state.capacity} slots · ${state.scheduling}` : "";
  const chat = state.chats.find((c) => c.id === current);
  $("chat-header").hidden = $("composer").hidden = !chat;
  const box = $("messages");
  box.replaceChildren();
  if (!chat) return;
  if (document.activeElement !== $("chat-title")) $("chat-title").value = chat.title;
  for (const msg of chat.messages) {
    const wrap = el("article", "msg " + msg.role);
    if (msg.role === "assistant") {
      const job = state.jobs.find((j) => j.id === msg.job) || {};
      if (job.thinking) {
        const details = el("details", "thinking");
        details.appendChild(el("summary", "", "Reasoning"));
        details.appendChild(el("pre", "", job.thinking));
        wrap.appendChild(details);
      }
      wrap.appendChild(el("div", "content", msg.content || (msg.status === "queued" ? "Waiting for the model…" : "")));
      const meta = [msg.status];
      if (job.output_tokens) meta.push(`${job.output_tokens} tokens`);
      if (job.decode_tps) meta.push(`${job.decode_tps.toFixed(1)} tok/s`);
      wrap.appendChild(el("footer", "meta", meta.join(" · ")));
    } else {
      wrap.appendChild(el("div", "content", msg.content));
    }
    box.appendChild(wrap);
  }
  box.scrollTop = box.scrollHeight;
}

async function refresh() {
  try {
    const res = await fetch("/api/state");
    state = await res.json();
    if (!current && state.chats.length) current = state.chats[state.chats.length - 1].id;
    render();
  } catch (err) {
    $("banner").hidden = false;
    $("banner").textContent = "The local server is not answering.";
  }
}

$("new-chat").addEventListener("click", async () => { current = (await post({ action: "create" })).id; refresh(); });
$("delete-chat").addEventListener("click", async () => {
  try { await post({ action: "delete", chat: current }); current = null; } catch (err) { alert(err.message); }
  refresh();
});
$("chat-title").addEventListener("change", async (ev) => {
  try { await post({ action: "rename", chat: current, title: ev.target.value }); } catch (err) { alert(err.message); }
  refresh();
});
$("composer").addEventListener("submit", async (ev) => {
  ev.preventDefault();
  const text = $("prompt").value;
  if (!text.trim() || !current) return;
  try { await post({ action: "send", chat: current, id: hexId(), text }); $("prompt").value = ""; } catch (err) { alert(err.message); }
  refresh();
});
refresh();
setInterval(refresh, 1000);
